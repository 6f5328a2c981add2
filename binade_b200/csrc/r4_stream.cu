// Batch-1 fused R4 matvec, streaming version: every warp owns a contiguous range of weight rows
// and pulls them through its own ring of shared-memory stages with 1-D bulk copies
// (cp.async.bulk + mbarrier complete_tx), so decode never waits on HBM latency and no warp waits
// on another. The warp walks its rows RW at a time to reuse the x registers.
//
//   stage   RW rows x KC tiles: raw [RW][KC*128] bytes, codes [RW][KC*64] bytes
//   lane l  owns weights 128t + 4l + j of every tile (the documented summation order)
//   x       whole vector as fp32 in shared memory; pair table (see r4_kernels.cu) per lane
//
// Requires K % 16 == 0 (bulk copies need 16-byte aligned row segments) and an x vector that fits
// shared memory beside the table and the rings; other shapes take the plain-load kernel.
#include <stdlib.h>

#include "common.cuh"

namespace bn {

constexpr int ST_KC = 8;             // tiles per stage
constexpr int ST_LUT_BYTES = 256 * 256;  // entry i of lane l at i * 256 + l * 4
constexpr uint32_t ST_SPIN_LIMIT = 1u << 24;

__device__ int g_stream_error;  // set when a bounded wait gives up; read by bn_device_status()

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after ST_SPIN_LIMIT polls and reports through g_stream_error.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < ST_SPIN_LIMIT; i++)
    if (mbar_try_wait(bar, parity)) return true;
  atomicExch(&g_stream_error, 1);
  return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
struct StreamArgs {
  bn_r4 w;
  const uint16_t *x;
  uint16_t *y;
  int64_t N, K;
  int T;
  int stages;  // ring depth per warp
};

// Escapes of one flagged lane word, in weight order across the warp: OR-masks for the two
// BF16x2 words (exponent bits of the code-15 weights, from the row's escape cursor) and the
// tile's escape count. Nearly every flagged tile holds its escapes in a single lane: that lane
// reads them straight from the cursor and the warp learns the count with one shuffle; otherwise
// a ballot scan orders the lanes. Out of line on purpose: flagged tiles are rare and the hot
// loop has to stay within the instruction cache. Whole warp calls it.
__device__ __noinline__ uint3 escape_patch(uint32_t c, const uint8_t *__restrict__ esc, uint32_t epos) {
  const uint32_t hit = c & (c >> 1) & (c >> 2) & (c >> 3) & 0x1111u;  // bit 4j: code j == 15
  const uint32_t lanes = __ballot_sync(BN_FULL, hit != 0);
  uint32_t q = epos, tot;
  if ((lanes & (lanes - 1)) == 0) {  // zero or one lane
    tot = __shfl_sync(BN_FULL, (uint32_t)__popc(hit), lanes ? __ffs(lanes) - 1 : 0);
  } else {
    uint32_t pre;
    warp_scan_small(__popc(hit), lanemask_lt(), pre, tot);
    q += pre;
  }
  uint32_t o01 = 0, o23 = 0;
  if (hit & 0x0001u) o01 |= (uint32_t)esc[q++] << 7;
  if (hit & 0x0010u) o01 |= (uint32_t)esc[q++] << 23;
  if (hit & 0x0100u) o23 |= (uint32_t)esc[q++] << 7;
  if (hit & 0x1000u) o23 |= (uint32_t)esc[q++] << 23;
  return make_uint3(o01, o23, tot);
}

// One stage (nt <= ST_KC tiles) of RWG rows: decode and accumulate. `stage` points at this
// lane's raw bytes of row 0 (rows ST_KC*128 apart), `codes` at its code word of row 0 (rows
// ST_KC*64 apart); xs is this lane's slice of x for the stage's first tile; lut is this lane's
// column of the pair table. The tile loop is unrolled by two only: the whole hot loop must fit
// the instruction cache.
template <int RWG>
__device__ __forceinline__ void consume_stage(const uint8_t *stage, const uint8_t *codes, const float *xs, const uint8_t *lut, int nt, int klim, const uint32_t (&fbits)[RWG], uint32_t fany, const uint8_t *__restrict__ esc, uint32_t (&epos)[RWG], float (&acc)[RWG]) {
  constexpr uint32_t RAW_ROW = ST_KC * 128, CODE_ROW = ST_KC * 64;
#pragma unroll 2
  for (int u = 0; u < nt; u++) {
    const float4 xv = *reinterpret_cast<const float4 *>(xs + u * BN_TILE);
    uint32_t w01[RWG], w23[RWG], c4[RWG];
#pragma unroll
    for (int i = 0; i < RWG; i++) {
      const uint32_t r4 = *reinterpret_cast<const uint32_t *>(stage + i * RAW_ROW + u * 128);
      c4[i] = *reinterpret_cast<const uint16_t *>(codes + i * CODE_ROW + u * 64);
      const uint32_t e01 = *reinterpret_cast<const uint32_t *>(lut + (c4[i] & 0xFFu) * 256u);
      const uint32_t e23 = *reinterpret_cast<const uint32_t *>(lut + (c4[i] & 0xFF00u));
      w01[i] = (__byte_perm(r4, 0u, 0x1100) & 0x807F807Fu) | e01;
      w23[i] = (__byte_perm(r4, 0u, 0x3322) & 0x807F807Fu) | e23;
    }
    if ((fany >> u) & 1u) {
#pragma unroll
      for (int i = 0; i < RWG; i++)
        if ((fbits[i] >> u) & 1u) {
          const uint3 p = escape_patch(c4[i], esc, epos[i]);
          w01[i] |= p.x, w23[i] |= p.y, epos[i] += p.z;
        }
    }
    if (u * BN_TILE < klim) {
#pragma unroll
      for (int i = 0; i < RWG; i++) {
        float s = acc[i];
        s = __fmaf_rn(__uint_as_float(w01[i] << 16), xv.x, s);
        s = __fmaf_rn(__uint_as_float(w01[i] & 0xFFFF0000u), xv.y, s);
        s = __fmaf_rn(__uint_as_float(w23[i] << 16), xv.z, s);
        s = __fmaf_rn(__uint_as_float(w23[i] & 0xFFFF0000u), xv.w, s);
        acc[i] = s;
      }
    }
  }
}

// WARPS: streaming warps per block; RW: rows walked together (a warp's last rows % RW rows are
// walked one at a time)
template <int WARPS, int RW>
__global__ void __launch_bounds__(WARPS * 32, 1) r4_stream_kernel(StreamArgs a) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  constexpr int THREADS = WARPS * 32;
  const uint32_t lane = lane_id(), warp = threadIdx.x >> 5;
  const int64_t K = a.K;
  const int T = a.T, S = a.stages;
  const int Tpad = T * BN_TILE;
  // shared memory map: pair table | x fp32 [T*128] | per-warp rings | mbarriers
  constexpr uint32_t RAW_ROW = ST_KC * 128, CODE_ROW = ST_KC * 64;
  constexpr uint32_t RAW_STAGE = RW * RAW_ROW, STAGE = RAW_STAGE + RW * CODE_ROW;
  uint8_t *const p_lut = smem_raw;
  float *const p_x = reinterpret_cast<float *>(smem_raw + ST_LUT_BYTES);
  uint8_t *const p_ring = smem_raw + ST_LUT_BYTES + (size_t)Tpad * 4 + (size_t)warp * S * STAGE;
  const uint32_t s_ring = smem_addr(p_ring);
  const uint32_t s_bar = smem_addr(smem_raw) + ST_LUT_BYTES + (uint32_t)Tpad * 4 + WARPS * (uint32_t)S * STAGE + warp * (uint32_t)S * 8;

  // this warp's rows: nfull groups of RW rows, then the remaining rows one per group
  const int64_t workers = (int64_t)gridDim.x * WARPS, me = (int64_t)blockIdx.x * WARPS + warp;
  const int64_t r_begin = a.N * me / workers, r_end = a.N * (me + 1) / workers;
  const int nrows = (int)(r_end - r_begin);
  const int nfull = nrows / RW, ngroups = nfull + (nrows - nfull * RW);
  const int nchunks = (T + ST_KC - 1) / ST_KC;

  if (lane == 0)
    for (int s = 0; s < S; s++) mbar_init(s_bar + s * 8, 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  __syncwarp();

  // producer side: next (group, chunk) to fetch and the ring slot it goes to
  int pg = 0, pc = 0, ps = 0;
  auto issue = [&]() {
    if (pg >= ngroups) return;
    const int r0 = pg < nfull ? pg * RW : nfull * RW + (pg - nfull);
    const int nlive = pg < nfull ? RW : 1;
    const int t0 = pc * ST_KC, nt = min(ST_KC, T - t0);
    const uint32_t raw_bytes = (uint32_t)min((int64_t)nt * BN_TILE, K - (int64_t)t0 * BN_TILE), code_bytes = (uint32_t)nt * 64u;
    const uint32_t slot = s_ring + (uint32_t)ps * STAGE, bar = s_bar + (uint32_t)ps * 8;
    if (lane == 0) mbar_expect_tx(bar, (uint32_t)nlive * (raw_bytes + code_bytes));
    __syncwarp();
    const int64_t row = r_begin + r0;
    if ((int)lane < nlive) {
      bulk_g2s(slot + lane * RAW_ROW, a.w.raw + (row + lane) * K + (int64_t)t0 * BN_TILE, raw_bytes, bar);
    } else if ((int)lane >= 16 && (int)lane < 16 + nlive) {
      const uint32_t i = lane - 16;
      bulk_g2s(slot + RAW_STAGE + i * CODE_ROW, a.w.codes + ((row + i) * T + t0) * 32, code_bytes, bar);
    }
    if (++pc == nchunks) pc = 0, pg++;
    if (++ps == S) ps = 0;
  };
  for (int s = 0; s < S; s++) issue();

  // while the first stages fly: pair table and x into shared memory (whole block)
  {
    __shared__ uint32_t t16[16];
    if (threadIdx.x < 16) t16[threadIdx.x] = threadIdx.x == 15 ? 0u : (uint32_t)a.w.table[threadIdx.x];
    // x: 8 BF16 values (16 bytes) per load, every load of the block in flight at once
    const uint4 *x8 = reinterpret_cast<const uint4 *>(a.x);
    for (int i = threadIdx.x; i < Tpad / 8; i += THREADS) {
      uint4 v = make_uint4(0, 0, 0, 0);
      if ((int64_t)i * 8 < K) v = __ldg(x8 + i);  // K % 16 == 0: a group of 8 is all in or all out
      float4 lo, hi;
      lo.x = __uint_as_float(v.x << 16), lo.y = __uint_as_float(v.x & 0xFFFF0000u), lo.z = __uint_as_float(v.y << 16), lo.w = __uint_as_float(v.y & 0xFFFF0000u);
      hi.x = __uint_as_float(v.z << 16), hi.y = __uint_as_float(v.z & 0xFFFF0000u), hi.z = __uint_as_float(v.w << 16), hi.w = __uint_as_float(v.w & 0xFFFF0000u);
      reinterpret_cast<float4 *>(p_x)[2 * i] = lo;
      reinterpret_cast<float4 *>(p_x)[2 * i + 1] = hi;
    }
    __syncthreads();
    uint32_t *lut = reinterpret_cast<uint32_t *>(p_lut);
    for (uint32_t i = threadIdx.x; i < 256 * 32; i += THREADS) {
      const uint32_t code = i >> 5, l = i & 31;
      lut[code * 64 + l] = (t16[code & 15] << 7) | (t16[code >> 4] << 23);
    }
    __syncthreads();
  }

  const uint8_t *lut_lane = p_lut + lane * 4;
  int cs = 0;           // consumer slot
  uint32_t phases = 0;  // bit s: parity to wait for on slot s
  // flag bytes (one 32-tile group per row at a time) and escape cursors are fetched one step
  // ahead of their use, so their global-memory latency hides behind the previous tiles
  auto group_row = [&](int g) { return g < nfull ? g * RW : nfull * RW + (g - nfull); };
  uint32_t pf_flag[RW], pf_epos[RW];
  auto prefetch_flags = [&](int g, int f) {
    const int r0 = group_row(g), live = g < nfull ? RW : 1;
#pragma unroll
    for (int i = 0; i < RW; i++) {
      const int64_t r = r_begin + r0 + min(i, live - 1);
      pf_flag[i] = f * 32 + (int)lane < T ? (uint32_t)a.w.flags[r * T + f * 32 + lane] : 0u;
    }
  };
  auto prefetch_epos = [&](int g) {
    const int r0 = group_row(g), live = g < nfull ? RW : 1;
#pragma unroll
    for (int i = 0; i < RW; i++) pf_epos[i] = a.w.row_esc[r_begin + r0 + min(i, live - 1)];
  };
  if (ngroups > 0) prefetch_flags(0, 0), prefetch_epos(0);
  const int fgroups = (T + 31) / 32;
  for (int g = 0; g < ngroups; g++) {
    const bool wide = g < nfull;
    const int64_t row = r_begin + group_row(g);
    float acc[RW];
    uint32_t epos[RW], fmask[RW];
#pragma unroll
    for (int i = 0; i < RW; i++) acc[i] = 0.0f, epos[i] = pf_epos[i], fmask[i] = 0u;
    if (g + 1 < ngroups) prefetch_epos(g + 1);
    for (int c = 0; c < nchunks; c++) {
      const int t0 = c * ST_KC, nt = min(ST_KC, T - t0);
      if ((t0 & 31) == 0) {
        const int f = t0 >> 5;
#pragma unroll
        for (int i = 0; i < RW; i++) {
          const uint32_t m = __ballot_sync(BN_FULL, pf_flag[i] != 0);
          fmask[i] = (wide || i == 0) ? m : 0u;
        }
        if (f + 1 < fgroups) prefetch_flags(g, f + 1);
        else if (g + 1 < ngroups) prefetch_flags(g + 1, 0);
      }
      if (!mbar_wait(s_bar + (uint32_t)cs * 8, (phases >> cs) & 1u)) return;  // gave up: status flag is set
      phases ^= 1u << cs;
      const uint8_t *stage = p_ring + (size_t)cs * STAGE + lane * 4;
      const uint8_t *codes = p_ring + (size_t)cs * STAGE + RAW_STAGE + lane * 2;
      const float *xs = p_x + (size_t)t0 * BN_TILE + lane * 4;
      const int klim = (int)min((int64_t)ST_KC * BN_TILE, K - (int64_t)t0 * BN_TILE) - (int)lane * 4;  // columns left for this lane
      if (wide) {
        uint32_t fbits[RW], fany = 0;
#pragma unroll
        for (int i = 0; i < RW; i++) {
          fbits[i] = (fmask[i] >> (t0 & 31)) & ((1u << ST_KC) - 1u);
          fany |= fbits[i];
        }
        consume_stage<RW>(stage, codes, xs, lut_lane, nt, klim, fbits, fany, a.w.esc, epos, acc);
      } else {
        uint32_t fb1[1] = {(fmask[0] >> (t0 & 31)) & ((1u << ST_KC) - 1u)}, ep1[1] = {epos[0]};
        float ac1[1] = {acc[0]};
        consume_stage<1>(stage, codes, xs, lut_lane, nt, klim, fb1, fb1[0], a.w.esc, ep1, ac1);
        epos[0] = ep1[0], acc[0] = ac1[0];
      }
      __syncwarp();
      issue();  // refill the slot just drained
      if (++cs == S) cs = 0;
    }
    float mine = 0.0f;
#pragma unroll
    for (int i = 0; i < RW; i++) {
      float s = acc[i];
#pragma unroll
      for (int o = 16; o >= 1; o >>= 1) s = s + __shfl_xor_sync(BN_FULL, s, o);
      if ((int)lane == i) mine = s;
    }
    if ((int)lane < (wide ? RW : 1)) a.y[row + lane] = f32_to_bf16_bits(mine);
  }
}

static int stream_sms() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

template <int WARPS, int RW>
static int launch_stream(StreamArgs a, cudaStream_t s) {
  const size_t fixed = ST_LUT_BYTES + (size_t)a.T * BN_TILE * 4 + 64;
  const size_t stage = (size_t)RW * ST_KC * 192;
  const size_t limit = 227 * 1024;
  if (fixed + WARPS * 2 * (stage + 8) > limit) return -1;  // does not fit: caller falls back
  int stages = (int)((limit - fixed) / (WARPS * (stage + 8)));
  if (stages > 6) stages = 6;
  a.stages = stages;
  const size_t smem = fixed + (size_t)WARPS * stages * (stage + 8);
  auto kern = r4_stream_kernel<WARPS, RW>;
  BN_CUDA(allow_smem(kern, smem));
  int64_t blocks = stream_sms();
  const int64_t need = (a.N + WARPS - 1) / WARPS;
  if (blocks > need) blocks = need;
  kern<<<(unsigned)blocks, WARPS * 32, smem, s>>>(a);
  return launched("r4_stream_kernel");
}

// Streaming warps per block: 8, or 12 with BINADE_B200_STREAM_WARPS=12 (an experiment knob).
static int stream_warps() {
  static int n = 0;
  if (!n) {
    const char *e = getenv("BINADE_B200_STREAM_WARPS");
    n = (e && atoi(e) == 12) ? 12 : 8;
  }
  return n;
}

// Returns -1 when the shape is outside what the streaming kernel covers.
int stream_matvec(const bn_r4 *w, const uint16_t *x, int64_t N, int64_t K, uint16_t *y, cudaStream_t s) {
  const int64_t T = tiles(K);
  if (K % 16 || N < 1) return -1;
  StreamArgs a{};
  a.w = *w, a.x = x, a.y = y, a.N = N, a.K = K, a.T = (int)T;
  const bool wide = N / ((int64_t)stream_sms() * 8) >= 8;  // enough rows per warp to walk 4 at a time
  if (!wide) return launch_stream<8, 2>(a, s);
  if (stream_warps() == 12) {
    const int e = launch_stream<12, 4>(a, s);
    if (e >= 0) return e;
  }
  return launch_stream<8, 4>(a, s);
}

}  // namespace bn

extern "C" int bn_device_status(int *status) {
  if (!status) return bn::fail(BN_ERR_ARG, "bn_device_status: null pointer");
  BN_CUDA(cudaMemcpyFromSymbol(status, bn::g_stream_error, sizeof(int)));
  return BN_OK;
}

