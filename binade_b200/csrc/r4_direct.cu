// Batch-1 fused R4 matvec, register-pipelined version: every warp owns a contiguous range of
// weight rows, walks them RW at a time and loads raw bytes and code words straight from global
// memory into registers, one batch of BT tiles ahead of the batch it is decoding. There is no
// shared-memory staging of the weights and therefore no per-stage bookkeeping: the only shared
// data are x (BF16) and the per-lane pair table.
//
//   lane l  owns weights 128t + 4l + j of every tile (the documented summation order)
//   x       whole vector as BF16 in shared memory, multiplied with fma.rn.f32.bf16
//   table   256-entry pair table (code byte -> two exponents placed in a BF16x2 word), one column
//           per lane (entry i of lane l at i*256 + l*4), on a 64 KB boundary of the shared window
//           so that a lookup address is one byte permute of the code word into a per-lane base
//
// Needs K % 4 == 0 only (a lane's four raw bytes are one aligned 32-bit load).
#include "common.cuh"

namespace bn {
namespace {

constexpr uint32_t DR_BASE_MAX = 2048;  // the dynamic shared window starts below this address

__device__ __forceinline__ uint32_t ldg_u32(const uint8_t *p) {
  uint32_t v;
  asm("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_u16(const uint8_t *p) {
  uint16_t v;
  asm("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return v;
}
// x and the table never change after the block-wide barrier that publishes them; `ready` is a
// value produced after that barrier, so no read can move above it.
__device__ __forceinline__ uint32_t lut_read(uint32_t addr, uint32_t ready) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr), "r"(ready));
  return v;
}
template <int OFF>
__device__ __forceinline__ uint2 x_read(uint32_t addr, uint32_t ready) {
  uint2 v;
  asm("ld.shared.v2.u32 {%0, %1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(OFF), "r"(ready));
  return v;
}
// acc += w.lo * x.lo; acc += w.hi * x.hi with BF16 factors widened exactly (two fused ops).
__device__ __forceinline__ float fma2_bf16(uint32_t w, uint32_t x, float acc) {
  asm("{\n\t.reg .b16 wl, wh, xl, xh;\n\t"
      "mov.b32 {wl, wh}, %1;\n\t"
      "mov.b32 {xl, xh}, %2;\n\t"
      "fma.rn.f32.bf16 %0, wl, xl, %0;\n\t"
      "fma.rn.f32.bf16 %0, wh, xh, %0;\n\t}"
      : "+f"(acc)
      : "r"(w), "r"(x));
  return acc;
}

// Escapes of one flagged lane word (see r4_stream.cu): single-lane case inline, general case a
// ballot scan out of line. Whole warp calls it.
__device__ __noinline__ uint3 escape_scan(uint32_t hit, const uint8_t *__restrict__ esc, uint32_t epos) {
  uint32_t pre, tot;
  warp_scan_small(__popc(hit), lanemask_lt(), pre, tot);
  uint32_t q = epos + pre, o01 = 0, o23 = 0;
  if (hit & 0x0001u) o01 |= (uint32_t)esc[q++] << 7;
  if (hit & 0x0010u) o01 |= (uint32_t)esc[q++] << 23;
  if (hit & 0x0100u) o23 |= (uint32_t)esc[q++] << 7;
  if (hit & 0x1000u) o23 |= (uint32_t)esc[q++] << 23;
  return make_uint3(o01, o23, tot);
}
__device__ __forceinline__ void escape_patch(uint32_t c, const uint8_t *__restrict__ esc, uint32_t &epos, uint32_t &w01, uint32_t &w23) {
  const uint32_t hit = c & (c >> 1) & (c >> 2) & (c >> 3) & 0x1111u;  // bit 4j: code j == 15
  const uint32_t lanes = __ballot_sync(BN_FULL, hit != 0);
  if ((lanes & (lanes - 1)) == 0) {  // one lane (or none)
    if (hit) {
      uint32_t q = epos;
      if (hit & 0x0001u) w01 |= (uint32_t)esc[q++] << 7;
      if (hit & 0x0010u) w01 |= (uint32_t)esc[q++] << 23;
      if (hit & 0x0100u) w23 |= (uint32_t)esc[q++] << 7;
      if (hit & 0x1000u) w23 |= (uint32_t)esc[q] << 23;
    }
    epos += __shfl_sync(BN_FULL, (uint32_t)__popc(hit), __ffs(lanes | 0x80000000u) - 1);
  } else {
    const uint3 p = escape_scan(hit, esc, epos);
    w01 |= p.x, w23 |= p.y, epos += p.z;
  }
}

// One lane word: raw bytes + codes -> two BF16x2 words (escapes not applied).
__device__ __forceinline__ void decode_word(uint32_t r4, uint32_t c4, uint32_t lut, uint32_t ready, uint32_t &w01, uint32_t &w23) {
  w01 = (__byte_perm(r4, 0u, 0x1100) & 0x807F807Fu) | lut_read(__byte_perm(c4, lut, 0x7604), ready);  // lut + code byte 0 * 256
  w23 = (__byte_perm(r4, 0u, 0x3322) & 0x807F807Fu) | lut_read(__byte_perm(c4, lut, 0x7614), ready);  // lut + code byte 1 * 256
}

struct DirectArgs {
  bn_r4 w;
  const uint16_t *x;
  uint16_t *y, *y2;
  int64_t N, K;
  int T;
  uint32_t smem;
  const uint32_t *xi, *ei;  // expert gather (blockIdx.y = slot), nullptr: plain matvec
  int64_t RS, R0, split;
};

// A batch of BT full tiles of RWG rows held in registers.
template <int RWG, int BT>
struct Batch {
  uint32_t r[RWG][BT], c[RWG][BT];
};

template <int RWG, int BT>
__device__ __forceinline__ void load_batch(Batch<RWG, BT> &b, const uint8_t *const (&raw)[RWG], const uint8_t *const (&codes)[RWG], int tile) {
#pragma unroll
  for (int i = 0; i < RWG; i++)
#pragma unroll
    for (int u = 0; u < BT; u++) {
      b.r[i][u] = ldg_u32(raw[i] + (size_t)(tile + u) * 128);
      b.c[i][u] = ldg_u16(codes[i] + (size_t)(tile + u) * 64);
    }
}

// Decode + accumulate a batch. fbits[i]: flag bits of row i, tile `tile0` at bit 0. A batch
// without a flagged tile is one straight line of code; otherwise every word tests its flag.
template <int RWG, int BT>
__device__ __forceinline__ void compute_batch(const Batch<RWG, BT> &b, uint32_t xs, uint32_t lut, uint32_t ready, const uint32_t (&fbits)[RWG], const uint8_t *__restrict__ esc, uint32_t (&epos)[RWG], float (&acc)[RWG]) {
  uint32_t any = 0;
#pragma unroll
  for (int i = 0; i < RWG; i++) any |= fbits[i];
  if (!(any & ((1u << BT) - 1u))) {
#pragma unroll
    for (int u = 0; u < BT; u++) {
      const uint2 xv = u == 0 ? x_read<0>(xs, ready) : u == 1 ? x_read<256>(xs, ready) : u == 2 ? x_read<512>(xs, ready) : u == 3 ? x_read<768>(xs, ready) : u == 4 ? x_read<1024>(xs, ready) : u == 5 ? x_read<1280>(xs, ready) : u == 6 ? x_read<1536>(xs, ready) : x_read<1792>(xs, ready);
#pragma unroll
      for (int i = 0; i < RWG; i++) {
        uint32_t w01, w23;
        decode_word(b.r[i][u], b.c[i][u], lut, ready, w01, w23);
        acc[i] = fma2_bf16(w23, xv.y, fma2_bf16(w01, xv.x, acc[i]));
      }
    }
  } else {
#pragma unroll
    for (int u = 0; u < BT; u++) {
      const uint2 xv = u == 0 ? x_read<0>(xs, ready) : u == 1 ? x_read<256>(xs, ready) : u == 2 ? x_read<512>(xs, ready) : u == 3 ? x_read<768>(xs, ready) : u == 4 ? x_read<1024>(xs, ready) : u == 5 ? x_read<1280>(xs, ready) : u == 6 ? x_read<1536>(xs, ready) : x_read<1792>(xs, ready);
#pragma unroll
      for (int i = 0; i < RWG; i++) {
        uint32_t w01, w23;
        decode_word(b.r[i][u], b.c[i][u], lut, ready, w01, w23);
        if ((fbits[i] >> u) & 1u) escape_patch(b.c[i][u], esc, epos[i], w01, w23);
        acc[i] = fma2_bf16(w23, xv.y, fma2_bf16(w01, xv.x, acc[i]));
      }
    }
  }
}

// RWG rows from tile 0 to the end of the row; rows are `rows[i]` (storage rows).
template <int RWG, int BT>
__device__ __forceinline__ void walk_rows(const DirectArgs &a, const int64_t (&rows)[RWG], uint32_t x_lane, uint32_t lut, uint32_t ready, float (&acc)[RWG]) {
  const uint32_t lane = lane_id();
  const int T = a.T;
  const int64_t K = a.K;
  const int full_tiles = (int)(K >> 7);  // tiles in which every lane holds weights
  const uint8_t *raw[RWG], *codes[RWG];
  uint32_t epos[RWG];
#pragma unroll
  for (int i = 0; i < RWG; i++) {
    raw[i] = a.w.raw + rows[i] * K + lane * 4;
    codes[i] = reinterpret_cast<const uint8_t *>(a.w.codes) + (rows[i] * T) * 64 + lane * 2;
    epos[i] = a.w.row_esc[rows[i]];
    acc[i] = 0.0f;
  }
  const int nb = full_tiles / BT;
  Batch<RWG, BT> cur, nxt;
  if (nb > 0) load_batch(cur, raw, codes, 0);
  uint32_t fmask[RWG] = {};
#pragma unroll 2
  for (int bi = 0; bi < nb; bi++) {
    const int tile = bi * BT;
    if (bi + 1 < nb) load_batch(nxt, raw, codes, tile + BT);
    if ((tile & 31) == 0) {
#pragma unroll
      for (int i = 0; i < RWG; i++) fmask[i] = __ballot_sync(BN_FULL, tile + (int)lane < T && a.w.flags[rows[i] * T + tile + lane] != 0);
    }
    uint32_t fbits[RWG];
#pragma unroll
    for (int i = 0; i < RWG; i++) fbits[i] = fmask[i] >> (tile & 31);
    compute_batch<RWG, BT>(cur, x_lane + (uint32_t)tile * 256u, lut, ready, fbits, a.w.esc, epos, acc);
    cur = nxt;
  }
  // the tiles left over (fewer than BT full ones, and a partial last tile), one at a time
  for (int tile = nb * BT; tile < T; tile++) {
    const bool in = (int64_t)tile * BN_TILE + lane * 4 < K;
    if ((tile & 31) == 0) {
#pragma unroll
      for (int i = 0; i < RWG; i++) fmask[i] = __ballot_sync(BN_FULL, tile + (int)lane < T && a.w.flags[rows[i] * T + tile + lane] != 0);
    }
    const uint2 xv = x_read<0>(x_lane + (uint32_t)tile * 256u, ready);
#pragma unroll
    for (int i = 0; i < RWG; i++) {
      const uint32_t r4 = in ? ldg_u32(raw[i] + (size_t)tile * 128) : 0u;
      const uint32_t c4 = ldg_u16(codes[i] + (size_t)tile * 64);
      uint32_t w01, w23;
      decode_word(r4, c4, lut, ready, w01, w23);
      if ((fmask[i] >> (tile & 31)) & 1u) escape_patch(c4, a.w.esc, epos[i], w01, w23);
      const float s = fma2_bf16(w23, xv.y, fma2_bf16(w01, xv.x, acc[i]));
      acc[i] = in ? s : acc[i];
    }
  }
}

}  // namespace

namespace {

// WARPS warps per block, one block per SM; RW rows walked together; BT tiles per register batch.
// Shared window by absolute address: [base, 64K) x as BF16 [T*128]; [64K, 128K) the pair table.
template <int WARPS, int RW, int BT>
__global__ void __launch_bounds__(WARPS * 32, 1) r4_direct_kernel(DirectArgs a) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  constexpr int THREADS = WARPS * 32;
  const uint32_t lane = lane_id(), warp = threadIdx.x >> 5;
  const int64_t K = a.K;
  const int T = a.T;
  const uint32_t base = smem_addr(smem_raw);
  const uint32_t x_at = (base + 15u) & ~15u;
  if (base > DR_BASE_MAX || x_at + (uint32_t)T * 256u > 65536u || a.smem < 131072u - base) return;  // the host checked the same layout
  const int64_t slot = blockIdx.y;
  if (a.ei && a.ei[slot] == BN_NO_EXPERT) return;  // a padding slot
  const int64_t row0 = a.ei ? (int64_t)a.ei[slot] * a.RS + a.R0 : 0;  // storage row of output row 0
  {
    const uint4 *x8 = reinterpret_cast<const uint4 *>(a.x + (a.ei ? (int64_t)a.xi[slot] * K : 0));
    const uint32_t *x2 = reinterpret_cast<const uint32_t *>(x8);
    uint32_t *dst = reinterpret_cast<uint32_t *>(smem_raw + (x_at - base));
    if ((K & 7) == 0 && (reinterpret_cast<uintptr_t>(x8) & 15) == 0) {
      for (int i = threadIdx.x; i < T * 16; i += THREADS) reinterpret_cast<uint4 *>(dst)[i] = (int64_t)i * 8 < K ? __ldg(x8 + i) : make_uint4(0, 0, 0, 0);
    } else {  // K % 4 == 0 only, or an input row that is not 16-byte aligned: two values per load
      for (int i = threadIdx.x; i < T * 64; i += THREADS) dst[i] = (int64_t)i * 2 < K ? __ldg(x2 + i) : 0u;
    }
    uint32_t *lut = reinterpret_cast<uint32_t *>(smem_raw + (65536u - base));
    for (uint32_t i = threadIdx.x; i < 256 * 32; i += THREADS) {
      const uint32_t code = i >> 5, l = i & 31, c0 = code & 15, c1 = code >> 4;
      const uint32_t e0 = c0 == 15 ? 0u : __ldg(a.w.table + c0), e1 = c1 == 15 ? 0u : __ldg(a.w.table + c1);
      lut[code * 64 + l] = (e0 << 7) | (e1 << 23);
    }
    __syncthreads();
  }
  uint32_t ready;
  asm volatile("mov.u32 %0, 0;" : "=r"(ready)::"memory");  // after the barrier: orders x / table reads
  const uint32_t lut_lane = 65536u + lane * 4, x_lane = x_at + lane * 8;

  const int64_t workers = (int64_t)gridDim.x * WARPS, me = (int64_t)blockIdx.x * WARPS + warp;
  const int64_t o_begin = a.N * me / workers, o_end = a.N * (me + 1) / workers;  // output rows of this warp
  auto store = [&](int64_t o, float v) {
    const uint16_t h = f32_to_bf16_bits(v);
    if (a.split > 0 && o >= a.split) a.y2[slot * (a.N - a.split) + (o - a.split)] = h;
    else a.y[slot * (a.split > 0 ? a.split : a.N) + o] = h;
  };
  int64_t o = o_begin;
  for (; o + RW <= o_end; o += RW) {
    int64_t rows[RW];
    float acc[RW];
#pragma unroll
    for (int i = 0; i < RW; i++) rows[i] = row0 + o + i;
    walk_rows<RW, BT>(a, rows, x_lane, lut_lane, ready, acc);
    float mine = 0.0f;
#pragma unroll
    for (int i = 0; i < RW; i++) {
      float s = acc[i];
#pragma unroll
      for (int k = 16; k >= 1; k >>= 1) s = s + __shfl_xor_sync(BN_FULL, s, k);
      if ((int)lane == i) mine = s;
    }
    if ((int)lane < RW) store(o + lane, mine);
  }
  for (; o < o_end; o++) {
    int64_t rows[1] = {row0 + o};
    float acc[1];
    walk_rows<1, BT>(a, rows, x_lane, lut_lane, ready, acc);
    float s = acc[0];
#pragma unroll
    for (int k = 16; k >= 1; k >>= 1) s = s + __shfl_xor_sync(BN_FULL, s, k);
    if (lane == 0) store(o, s);
  }
}

int direct_sms() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

template <int WARPS, int RW, int BT>
int launch_direct(DirectArgs a, cudaStream_t s, int64_t slots) {
  if ((uint32_t)a.T * 256u + DR_BASE_MAX + 16u > 65536u) return -1;  // x does not fit below the table
  a.smem = 131072u;  // x + table; the window's start is below DR_BASE_MAX
  auto kern = r4_direct_kernel<WARPS, RW, BT>;
  BN_CUDA(allow_smem(kern, a.smem));
  int64_t blocks = (direct_sms() + slots - 1) / slots;
  const int64_t need = (a.N + WARPS - 1) / WARPS;
  if (blocks > need) blocks = need;
  kern<<<dim3((unsigned)blocks, (unsigned)slots), WARPS * 32, a.smem, s>>>(a);
  return launched("r4_direct_kernel");
}

int direct_any(DirectArgs a, cudaStream_t s, int64_t slots) {
  // 32 warps with short register batches measured best on long rows (K = 15360: 30 us against
  // 37 us with 24 warps); the launch bound of 1024 threads caps registers at 64
  return launch_direct<32, 2, 4>(a, s, slots);
}

}  // namespace

// Returns -1 when the shape is outside what this kernel covers (K % 4 != 0, or x too long for
// the shared window below the table: K > 31744).
int direct_matvec(const bn_r4 *w, const uint16_t *x, int64_t N, int64_t K, uint16_t *y, cudaStream_t s) {
  if (K % 4 || N < 1 || (reinterpret_cast<uintptr_t>(x) & 3) || (reinterpret_cast<uintptr_t>(w->raw) & 3)) return -1;  // 32-bit loads of x and of the raw bytes
  DirectArgs a{};
  a.w = *w, a.x = x, a.y = y, a.N = N, a.K = K, a.T = (int)tiles(K);
  return direct_any(a, s, 1);
}

int direct_gather(const bn_r4 *w, const uint16_t *x, const uint32_t *xi, const uint32_t *ei, int64_t G, int64_t n, int64_t K, int64_t RS, int64_t R0, int64_t split, uint16_t *y, uint16_t *y2, cudaStream_t s) {
  if (K % 4 || n < 1 || G < 1 || G > 65535 || (reinterpret_cast<uintptr_t>(x) & 3) || (reinterpret_cast<uintptr_t>(w->raw) & 3)) return -1;
  DirectArgs a{};
  a.w = *w, a.x = x, a.y = y, a.y2 = y2, a.N = n, a.K = K, a.T = (int)tiles(K);
  a.xi = xi, a.ei = ei, a.RS = RS, a.R0 = R0, a.split = split;
  return direct_any(a, s, G);
}

}  // namespace bn
