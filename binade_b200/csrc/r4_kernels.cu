// R4 kernels: dense decode, and the fused decode + product kernels (matvec, small-M rows,
// expert gather). One warp owns whole weight rows; lane l owns weights 128t + 4l + j of every
// tile t, which is both the layout of an R4 lane word (4 raw bytes + one uint16 of codes) and
// the documented summation order.
#include <stdlib.h>

#include "common.cuh"
#include "decode.cuh"
#include "oct.cuh"

namespace bn {

__device__ __forceinline__ float lo_f32(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float hi_f32(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// ---------------------------------------------------------------------------------------------
// R4 -> dense BF16
// ---------------------------------------------------------------------------------------------
constexpr int DEC_THREADS = 256;

__global__ void __launch_bounds__(DEC_THREADS) r4_decode_kernel(bn_r4 w, int64_t N, int64_t K, int T, int64_t NB, int64_t RS, int64_t R0, const uint32_t *__restrict__ ids, int64_t rows, uint16_t *__restrict__ out) {
  extern __shared__ uint32_t lut[];
  build_pair_lut(lut, w.table);
  __syncthreads();
  const uint32_t lane = lane_id(), lt = lanemask_lt();
  const uint32_t lut_lane = smem_addr(lut) + lane * 4;
  const int warps = DEC_THREADS / 32;
  for (int64_t orow = (int64_t)blockIdx.x * warps + (threadIdx.x >> 5); orow < N; orow += (int64_t)gridDim.x * warps) {
    const int64_t row = ids ? (int64_t)ids[orow] : (orow / NB) * RS + R0 + orow % NB;
    if (ids && row >= rows) {  // an id outside the table: a row of zeros
      for (int64_t c = lane; c < K; c += 32) out[orow * K + c] = 0;
      continue;
    }
    uint32_t epos = w.row_esc[row];
    const uint8_t *raw = w.raw + row * K;
    const uint16_t *codes = w.codes + row * T * 32;
    const uint8_t *flags = w.flags + row * T;
    uint2 *o = reinterpret_cast<uint2 *>(out + orow * K);
    for (int t0 = 0; t0 < T; t0 += 32) {
      const uint32_t fmask = __ballot_sync(BN_FULL, t0 + (int)lane < T && flags[t0 + lane] != 0);
      const int tn = min(32, T - t0);
#pragma unroll 4
      for (int u = 0; u < tn; u++) {
        const int t = t0 + u;
        const bool in = t * BN_TILE + (int)lane * 4 < K;
        uint32_t r = in ? ldg_stream_u32(raw + t * BN_TILE + lane * 4) : 0u;
        uint32_t c = ldg_stream_u16(codes + t * 32 + lane);
        uint32_t w01, w23;
        decode4(r, c, lut_lane, w01, w23);
        if ((fmask >> u) & 1u) apply_escapes(c, w.esc, epos, lt, w01, w23);
        if (in) o[t * 32 + lane] = make_uint2(w01, w23);
      }
    }
  }
}

// The same decode with eight threads per row (K % 16 == 0): a thread loads 16 raw bytes and 8
// bytes of code words of a tile with one load each, decodes 16 weights and stores 32 bytes, so a
// warp instruction moves four rows' worth; escapes by column streams when the matrix carries
// them. About a third of the instructions per weight of the kernel above.
template <bool COLS>
__global__ void __launch_bounds__(DEC_THREADS) r4_decode_wide_kernel(bn_r4 w, int64_t N, int64_t K, int T, int64_t NB, int64_t RS, int64_t R0, uint16_t *__restrict__ out) {
  constexpr int R = 4;
  using Geo = OctGeom<R>;
  extern __shared__ uint32_t lut[];
  build_pair_lut(lut, w.table);
  __syncthreads();
  const uint32_t lane = lane_id(), grp = lane >> 3, p = lane & 7u;
  OctSelf me;
  me.lane = lane, me.lane_hi = lane & ~7u, me.to_codes = 0, me.lut = smem_addr(lut) + lane * 4u, me.ready = 0;
  me.gmask = 0xFFu << (grp * 8u), me.ltg = me.gmask & lanemask_lt();
  me.esc = w.esc, me.esc_cap = w.n_esc + 1, me.esc_cols = w.esc_cols;
  const bool partial = (K & 127) != 0;
  const uint32_t pmax = (uint32_t)(K & 127) / 16u;
  const int warps = DEC_THREADS / 32;
  for (int64_t g = (int64_t)blockIdx.x * warps + (threadIdx.x >> 5); g * R < N; g += (int64_t)gridDim.x * warps) {
    const int64_t orow = g * R + grp;
    const bool valid = orow < N;
    const int64_t o = valid ? orow : N - 1;  // a slot past the last row decodes that row again and stores nothing
    const int64_t row = (o / NB) * RS + R0 + o % NB;
    const uint8_t *raw = w.raw + row * K + p * 16u;
    const uint8_t *codes = reinterpret_cast<const uint8_t *>(w.codes) + row * ((int64_t)T * 64) + p * 8u;
    const uint8_t *flags = w.flags + row * T;
    uint16_t *dst = out + o * K + p * 16u;
    uint32_t epos = __ldg(w.row_esc + row);
    EscWindow ew{};
    EscStream col[2]{};
    if constexpr (COLS) {
      const uint32_t starts = __ldg(reinterpret_cast<const uint32_t *>(w.col_esc + row * 16) + p);
      stream_open(col[0], w.esc_cols, epos + (starts & 0xFFFFu));
      stream_open(col[1], w.esc_cols, epos + (starts >> 16));
    } else {
      ew.base = epos & ~3u;
      ew.word = window_load(me.esc, me.esc_cap, ew.base + p * 4u);
    }
    uint32_t fm = 0;
    for (int t = 0; t < T; t++) {
      if ((t & 7) == 0) {  // the flag bytes of eight tiles, folded over the warp's four rows
        const uint32_t f = t + (int)p < T ? (uint32_t)__ldg(flags + t + p) : 0u;
        const uint32_t v = __ballot_sync(BN_FULL, f != 0);
        fm = (v | (v >> 8) | (v >> 16) | (v >> 24)) & 0xFFu;
      }
      const bool live = !(partial && t == T - 1) || p < pmax;
      const uint4 rr = live ? __ldcs(reinterpret_cast<const uint4 *>(raw + (int64_t)t * 128)) : make_uint4(0, 0, 0, 0);
      const uint2 c2 = __ldcs(reinterpret_cast<const uint2 *>(codes + (int64_t)t * 64));
      const uint32_t r4w[4] = {rr.x, rr.y, rr.z, rr.w}, cc[2] = {c2.x, c2.y};
      uint32_t wv[2 * R];
#pragma unroll
      for (int i = 0; i < R; i++) {
        const uint32_t c = (i & 1) ? cc[i >> 1] >> 16 : cc[i >> 1];
        wv[2 * i] = (__byte_perm(r4w[i], 0u, 0x1100) & 0x807F807Fu) | lds_u32(me.lut + ((c << 7) & 0x7F80u));
        wv[2 * i + 1] = (__byte_perm(r4w[i], 0u, 0x3322) & 0x807F807Fu) | lds_u32(me.lut + ((c >> 1) & 0x7F80u));
      }
      if ((fm >> (t & 7)) & 1u) {
        if constexpr (COLS) {
          const uint32_t h0 = hits15(cc[0]), h1 = hits15(cc[1]);
          if (h0) stream_patch<0>(h0, col[0], w.esc_cols, wv);
          if (h1) stream_patch<4>(h1, col[1], w.esc_cols, wv);
        } else {
          oct_patch<R>(epos, ew, wv, cc, me);
        }
      }
      if (valid && live) {
        uint4 *d = reinterpret_cast<uint4 *>(dst + (int64_t)t * 128);
        __stcs(d, make_uint4(wv[0], wv[1], wv[2], wv[3]));
        __stcs(d + 1, make_uint4(wv[4], wv[5], wv[6], wv[7]));
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Fused decode + product: Y[m, r] = sum_k X[m, k] W[r, k]
//   M   input rows held per pass (accumulators per weight row)
//   RW  weight rows a warp works on at once (reuses the x registers)
// x lives in shared memory as fp32, staged in chunks of KC tiles when M * K is large.
// ---------------------------------------------------------------------------------------------
constexpr int MV_THREADS = 512;  // launch bound; small matrices launch fewer warps per block

struct RowsArgs {
  bn_r4 w;
  const uint16_t *x;
  int64_t x_stride;
  const uint32_t *xi, *ei;  // per-slot input row / expert (gather only)
  int m;                    // input rows really present (<= M of the instantiation)
  int64_t n;                // weight rows per slot
  int64_t K;
  int T;
  int KC;  // tiles of x staged at a time
  int64_t RS, R0, split;
  uint16_t *y, *y2;
  int64_t y_stride;
};

template <int M, int RW, bool GATHER>
__global__ void __launch_bounds__(MV_THREADS) r4_rows_kernel(RowsArgs a) {
  constexpr int U = 4;  // tiles whose loads are issued before any is consumed
  extern __shared__ uint32_t smem[];
  uint32_t *lut = smem;
  float *xs = reinterpret_cast<float *>(smem + LUT_WORDS);  // [M][KC * 128]
  const uint32_t lane = lane_id(), lt = lanemask_lt(), warp = threadIdx.x >> 5;
  const uint32_t lut_lane = smem_addr(lut) + lane * 4;
  const int warps = blockDim.x >> 5;
  const int64_t K = a.K;
  const int T = a.T, KC = a.KC;
  const int xs_stride = KC * BN_TILE;

  int64_t row0 = 0;  // storage row of output row 0
  const uint16_t *x = a.x;
  int64_t g = 0;
  if (GATHER) {
    g = blockIdx.y;
    if (a.ei[g] == BN_NO_EXPERT) return;  // a padding slot
    row0 = (int64_t)a.ei[g] * a.RS + a.R0;
    x = a.x + (int64_t)a.xi[g] * a.x_stride;
  }
  build_pair_lut(lut, a.w.table);

  const bool one_chunk = KC >= T;
  const int64_t block_rows = (int64_t)warps * RW;
  const int64_t first_rb = (int64_t)blockIdx.x * block_rows;
  for (int64_t rb = first_rb; rb < a.n; rb += (int64_t)gridDim.x * block_rows) {
    float acc[RW][M];
    uint32_t epos[RW];
    const uint8_t *raw_row[RW];
    const uint16_t *code_row[RW];
    const uint8_t *flag_row[RW];
    bool live[RW];
#pragma unroll
    for (int i = 0; i < RW; i++) {
      const int64_t r = rb + (int64_t)warp * RW + i;
      live[i] = r < a.n;
      const int64_t srow = row0 + (live[i] ? r : 0);
      epos[i] = a.w.row_esc[srow];
      raw_row[i] = a.w.raw + srow * K + lane * 4;
      code_row[i] = a.w.codes + srow * T * 32 + lane;
      flag_row[i] = a.w.flags + srow * T;
#pragma unroll
      for (int m = 0; m < M; m++) acc[i][m] = 0.0f;
    }
    for (int tc = 0; tc < T; tc += KC) {
      // stage x[:, tc*128 ..) as fp32; absent rows and columns >= K hold zeros and are
      // never multiplied into a real output (see `in` and the store predicate)
      if (!one_chunk || rb == first_rb) {
        __syncthreads();
        for (int i = threadIdx.x; i < M * xs_stride; i += blockDim.x) {
          const int m = i / xs_stride, col = i - m * xs_stride;
          const int64_t k = (int64_t)tc * BN_TILE + col;
          xs[i] = (m < a.m && k < K) ? __uint_as_float((uint32_t)x[m * a.x_stride + k] << 16) : 0.0f;
        }
        __syncthreads();
      }
      const int tend = min(T, tc + KC);
      for (int t0 = tc; t0 < tend; t0 += 32) {
        uint32_t fmask[RW], fany = 0;
#pragma unroll
        for (int i = 0; i < RW; i++) {
          fmask[i] = __ballot_sync(BN_FULL, t0 + (int)lane < tend && flag_row[i][t0 + lane] != 0);
          fany |= fmask[i];
        }
        const int tn = min(32, tend - t0);
        for (int u0 = 0; u0 < tn; u0 += U) {
          uint32_t r4[U][RW], c4[U][RW];
#pragma unroll
          for (int uu = 0; uu < U; uu++) {
            const int t = t0 + u0 + uu;
            const bool in = u0 + uu < tn && (int64_t)t * BN_TILE + lane * 4 < K;
#pragma unroll
            for (int i = 0; i < RW; i++) {
              r4[uu][i] = in ? ldg_stream_u32(raw_row[i] + t * BN_TILE) : 0u;
              c4[uu][i] = in ? ldg_stream_u16(code_row[i] + t * 32) : 0u;
            }
          }
#pragma unroll
          for (int uu = 0; uu < U; uu++) {
            const int u = u0 + uu, t = t0 + u;
            if (u >= tn) break;
            const bool in = (int64_t)t * BN_TILE + lane * 4 < K;
            float wf[RW][4];
#pragma unroll
            for (int i = 0; i < RW; i++) {
              uint32_t w01, w23;
              decode4(r4[uu][i], c4[uu][i], lut_lane, w01, w23);
              if ((fany >> u) & 1u) {
                if ((fmask[i] >> u) & 1u) apply_escapes(c4[uu][i], a.w.esc, epos[i], lt, w01, w23);
              }
              wf[i][0] = lo_f32(w01), wf[i][1] = hi_f32(w01), wf[i][2] = lo_f32(w23), wf[i][3] = hi_f32(w23);
            }
            if (in) {
              const float *xt = xs + (t - tc) * BN_TILE + lane * 4;
#pragma unroll
              for (int m = 0; m < M; m++) {
                const float4 xv = *reinterpret_cast<const float4 *>(xt + m * xs_stride);
#pragma unroll
                for (int i = 0; i < RW; i++) {
                  float s = acc[i][m];
                  s = __fmaf_rn(wf[i][0], xv.x, s);
                  s = __fmaf_rn(wf[i][1], xv.y, s);
                  s = __fmaf_rn(wf[i][2], xv.z, s);
                  s = __fmaf_rn(wf[i][3], xv.w, s);
                  acc[i][m] = s;
                }
              }
            }
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < RW; i++) {
      float mine = 0.0f;
#pragma unroll
      for (int m = 0; m < M; m++) {
        float s = acc[i][m];
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) s = s + __shfl_xor_sync(BN_FULL, s, o);
        if ((int)lane == m) mine = s;
      }
      const int64_t r = rb + (int64_t)warp * RW + i;
      if (live[i] && (int)lane < a.m) {
        const uint16_t v = f32_to_bf16_bits(mine);
        if (GATHER) {
          if (a.split > 0 && r >= a.split)
            a.y2[g * (a.n - a.split) + (r - a.split)] = v;
          else
            a.y[g * (a.split > 0 ? a.split : a.n) + r] = v;
        } else {
          a.y[(int64_t)lane * a.y_stride + r] = v;
        }
      }
    }
  }
}

static int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

template <int M, int RW, bool GATHER>
static int launch_rows(RowsArgs a, int64_t G, cudaStream_t s) {
  // x chunk: whole K when it fits beside the table, else as many tiles as the budget holds
  int kc = a.T;
  const size_t budget = (M == 1 ? 192 : 96) * 1024;
  if ((size_t)M * kc * BN_TILE * 4 > budget) kc = (int)(budget / ((size_t)M * BN_TILE * 4));
  if (kc < 1) return fail(BN_ERR_ARG, "K too large for the fused rows kernel");
  a.KC = kc;
  const size_t smem = LUT_WORDS * 4 + (size_t)M * kc * BN_TILE * 4;
  auto kern = r4_rows_kernel<M, RW, GATHER>;
  BN_CUDA(allow_smem(kern, smem));
  // few rows: narrower blocks so that every SM gets work
  int threads = MV_THREADS;
  while (threads > 128 && (a.n * G + (threads / 32) * RW - 1) / ((threads / 32) * RW) < 2 * (int64_t)sm_count()) threads >>= 1;
  int per_sm = 1;
  BN_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, threads, smem));
  if (per_sm < 1) per_sm = 1;
  const int64_t block_rows = (int64_t)(threads / 32) * RW;
  int64_t blocks = (a.n + block_rows - 1) / block_rows;
  const int64_t cap = (int64_t)sm_count() * per_sm;
  if (blocks * G > cap) blocks = (cap + G - 1) / G;
  dim3 grid((unsigned)blocks, (unsigned)G);
  kern<<<grid, threads, smem, s>>>(a);
  return launched("r4_rows_kernel");
}

static int check_r4(const bn_r4 *w) {
  if (!w || !w->raw || !w->codes || !w->flags || !w->esc || !w->table || !w->row_esc) return fail(BN_ERR_ARG, "null R4 array");
  return BN_OK;
}

}  // namespace bn

using namespace bn;

extern "C" int bn_r4_decode(const bn_r4 *w, int64_t N, int64_t K, int64_t NB, int64_t RS, int64_t R0, uint16_t *out, void *stream) {
  if (int e = check_r4(w)) return e;
  if (!out || N < 0 || K <= 0 || NB <= 0) return fail(BN_ERR_ARG, "bn_r4_decode: bad size or null output");
  if (K % 4) return fail(BN_ERR_ARG, "R4 needs K % 4 == 0");
  if (N == 0) return BN_OK;
  const size_t smem = LUT_WORDS * 4;
  const int warps = DEC_THREADS / 32;
  if (K % 16 == 0 && !((reinterpret_cast<uintptr_t>(w->raw) | reinterpret_cast<uintptr_t>(w->codes) | reinterpret_cast<uintptr_t>(out)) & 15) && !((reinterpret_cast<uintptr_t>(w->esc) | reinterpret_cast<uintptr_t>(w->esc_cols) | reinterpret_cast<uintptr_t>(w->col_esc)) & 3)) {
    int64_t blocks = ((N + 3) / 4 + warps - 1) / warps;
    if (blocks > (int64_t)sm_count() * 7) blocks = (int64_t)sm_count() * 7;
    const bool cols = w->esc_cols && w->col_esc;
    auto kern = cols ? r4_decode_wide_kernel<true> : r4_decode_wide_kernel<false>;
    BN_CUDA(allow_smem(kern, smem));
    kern<<<(unsigned)blocks, DEC_THREADS, smem, (cudaStream_t)stream>>>(*w, N, K, (int)tiles(K), NB, RS, R0, out);
    return launched("r4_decode_wide_kernel");
  }
  BN_CUDA(allow_smem(r4_decode_kernel, smem));
  int64_t blocks = (N + warps - 1) / warps;
  if (blocks > (int64_t)sm_count() * 8) blocks = (int64_t)sm_count() * 8;
  r4_decode_kernel<<<(unsigned)blocks, DEC_THREADS, smem, (cudaStream_t)stream>>>(*w, N, K, (int)tiles(K), NB, RS, R0, nullptr, 0, out);
  return launched("r4_decode_kernel");
}

extern "C" int bn_r4_lookup(const bn_r4 *w, int64_t rows, const uint32_t *ids, int64_t n, int64_t K, uint16_t *out, void *stream) {
  if (int e = check_r4(w)) return e;
  if (!ids || !out || n < 0 || K <= 0 || rows < 0) return fail(BN_ERR_ARG, "bn_r4_lookup: bad size or null pointer");
  if (K % 4) return fail(BN_ERR_ARG, "R4 needs K % 4 == 0");
  if (n == 0) return BN_OK;
  const size_t smem = LUT_WORDS * 4;
  BN_CUDA(allow_smem(r4_decode_kernel, smem));
  const int warps = DEC_THREADS / 32;
  int64_t blocks = (n + warps - 1) / warps;
  if (blocks > (int64_t)sm_count() * 8) blocks = (int64_t)sm_count() * 8;
  r4_decode_kernel<<<(unsigned)blocks, DEC_THREADS, smem, (cudaStream_t)stream>>>(*w, n, K, (int)tiles(K), 1, 1, 0, ids, rows, out);
  return launched("r4_decode_kernel");
}

extern "C" int bn_r4_gather_grouped(const uint16_t *x, const bn_r4 *w, const uint32_t *xi, const uint32_t *seg, const uint32_t *order, int64_t E, int64_t G, int64_t max_per_expert, int64_t n, int64_t K, int64_t RS, int64_t R0, int64_t split, uint16_t *y, uint16_t *y2, void *stream) {
  if (int e = check_r4(w)) return e;
  if (!x || !xi || !seg || !order || !y || E < 1 || G < 0 || max_per_expert < 1 || n < 0 || K <= 0 || split < 0 || split >= (n > 0 ? n : 1)) return fail(BN_ERR_ARG, "bn_r4_gather_grouped: bad size or null pointer");
  if (split > 0 && !y2) return fail(BN_ERR_ARG, "bn_r4_gather_grouped: split needs y2");
  if (G == 0 || n == 0) return BN_OK;
  const int e = stream_gather_grouped(w, x, xi, seg, order, E, G, max_per_expert, n, K, RS, R0, split, y, y2, (cudaStream_t)stream);
  return e == -1 ? fail(BN_ERR_ARG, "bn_r4_gather_grouped: shape outside the streaming kernel (K % 16, row length, group count): use bn_r4_gather") : e;
}

extern "C" int bn_r4_rows(const uint16_t *x, int64_t x_stride, const bn_r4 *w, int64_t M, int64_t N, int64_t K, uint16_t *y, int64_t y_stride, void *stream) {
  if (int e = check_r4(w)) return e;
  if (!x || !y || N < 0 || K <= 0 || M < 1 || M > 16) return fail(BN_ERR_ARG, "bn_r4_rows: bad size (1 <= M <= 16) or null pointer");
  if (K % 4) return fail(BN_ERR_ARG, "R4 needs K % 4 == 0");
  if (N == 0) return BN_OK;
  RowsArgs a{};
  a.w = *w, a.x = x, a.x_stride = x_stride, a.n = N, a.K = K, a.T = (int)tiles(K), a.y = y, a.y_stride = y_stride;
  cudaStream_t s = (cudaStream_t)stream;
  a.m = (int)M;
  // the instantiation is the next power of two >= M: absent input rows are zeros in shared
  // memory and are never stored, so the weights stream once whatever M
  if (M == 1) {
    // the cp.async kernel (K % 16 == 0, 640 <= K <= 16384, aligned arrays); else, for long rows,
    // the register-pipelined kernel; else the bulk-copy kernel (K % 16 == 0); then whichever is left
    int e = oct_matvec(w, x, N, K, y, s);
    if (e == -1 && K >= 8192) e = direct_matvec(w, x, N, K, y, s);
    if (e == -1) e = stream_matvec(w, x, N, K, y, s);
    if (e == -1) e = direct_matvec(w, x, N, K, y, s);
    if (e >= 0) return e;
  }
  if (M == 1) return N >= 8192 ? launch_rows<1, 2, false>(a, 1, s) : launch_rows<1, 1, false>(a, 1, s);
  if (M <= 8) {
    const int e = stream_rows(w, x, x_stride, M, N, K, y, y_stride, s);
    if (e >= 0) return e;
  }
  if (M == 2) return launch_rows<2, 2, false>(a, 1, s);
  if (M <= 4) return launch_rows<4, 2, false>(a, 1, s);
  if (M <= 8) return launch_rows<8, 2, false>(a, 1, s);
  return launch_rows<16, 2, false>(a, 1, s);
}

extern "C" int bn_r4_rows_multi(const uint16_t *x, const bn_r4 *const *w, const int64_t *N, int count, int64_t K, uint16_t *const *y, void *stream) {
  if (!x || !w || !N || !y || count < 1 || count > 4 || K <= 0) return fail(BN_ERR_ARG, "bn_r4_rows_multi: 1..4 matrices, no null pointer");
  if (K % 4) return fail(BN_ERR_ARG, "R4 needs K % 4 == 0");
  for (int i = 0; i < count; i++) {
    if (int e = check_r4(w[i])) return e;
    if (!y[i] || N[i] < 0) return fail(BN_ERR_ARG, "bn_r4_rows_multi: bad size or null output");
  }
  // matrices with rows, in one launch when the shape allows it
  const bn_r4 *ws[4];
  int64_t Ns[4];
  uint16_t *ys[4];
  int n = 0;
  for (int i = 0; i < count; i++)
    if (N[i] > 0) ws[n] = w[i], Ns[n] = N[i], ys[n] = y[i], n++;
  if (n == 0) return BN_OK;
  const int e = oct_matvec_multi(ws, Ns, ys, n, x, K, (cudaStream_t)stream);
  if (e >= 0) return e;
  for (int i = 0; i < n; i++)
    if (int e1 = bn_r4_rows(x, K, ws[i], 1, Ns[i], K, ys[i], Ns[i], stream)) return e1;
  return BN_OK;
}

extern "C" int bn_r4_gather(const uint16_t *x, const bn_r4 *w, const uint32_t *xi, const uint32_t *ei, int64_t G, int64_t n, int64_t K, int64_t RS, int64_t R0, int64_t split, uint16_t *y, uint16_t *y2, void *stream) {
  if (int e = check_r4(w)) return e;
  if (!x || !xi || !ei || !y || G < 0 || n < 0 || K <= 0 || split < 0 || split >= (n > 0 ? n : 1)) return fail(BN_ERR_ARG, "bn_r4_gather: bad size or null pointer");
  if (split > 0 && !y2) return fail(BN_ERR_ARG, "bn_r4_gather: split needs y2");
  if (K % 4) return fail(BN_ERR_ARG, "R4 needs K % 4 == 0");
  if (G == 0 || n == 0) return BN_OK;
  if (G > 65535) return fail(BN_ERR_ARG, "bn_r4_gather: more than 65535 slots");
  {
    int e = oct_gather(w, x, xi, ei, G, n, K, RS, R0, split, y, y2, (cudaStream_t)stream);
    if (e == -1) e = stream_gather(w, x, xi, ei, G, n, K, RS, R0, split, y, y2, (cudaStream_t)stream);
    if (e == -1) e = direct_gather(w, x, xi, ei, G, n, K, RS, R0, split, y, y2, (cudaStream_t)stream);
    if (e >= 0) return e;
  }
  RowsArgs a{};
  a.w = *w, a.x = x, a.x_stride = K, a.xi = xi, a.ei = ei, a.n = n, a.K = K, a.T = (int)tiles(K);
  a.RS = RS, a.R0 = R0, a.split = split, a.y = y, a.y2 = y2, a.m = 1;
  return launch_rows<1, 1, true>(a, G, (cudaStream_t)stream);
}
