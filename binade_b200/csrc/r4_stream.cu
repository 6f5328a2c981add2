// Batch-1 fused R4 matvec, streaming version: every warp owns a contiguous range of weight rows
// and pulls them through its own ring of shared-memory stages with 1-D bulk copies
// (cp.async.bulk + mbarrier complete_tx), so decode never waits on HBM latency and no warp waits
// on another. The warp walks its rows RW at a time to reuse the x registers.
//
//   stage   RW rows x KC tiles: raw [RW][KC*128] bytes, codes [RW][KC*64] bytes
//   lane l  owns weights 128t + 4l + j of every tile (the documented summation order)
//   x       whole vector as BF16 in shared memory, multiplied with the mixed-precision
//           fma.rn.f32.bf16 (exact widening of both factors, one rounding of the sum)
//   table   pair table of r4_kernels.cu, entry i of lane l at i*256 + l*4, placed on a 64 KB
//           boundary of the shared window so that a lookup address is one byte permute of the
//           code word into a per-lane base
//
// Requires K % 16 == 0 (bulk copies need 16-byte aligned row segments) and an x vector that fits
// shared memory; other shapes take the plain-load kernel.
#include "common.cuh"

namespace bn {

constexpr uint32_t ST_SPIN_LIMIT = 1u << 24;
constexpr uint32_t ST_BASE_MAX = 2048;  // the dynamic shared window starts below this address

__device__ int g_stream_error;  // set when a bounded wait gives up; read by bn_device_status()

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Bounded wait: gives up after ST_SPIN_LIMIT polls and reports through g_stream_error. `token`
// receives a value the compiler cannot see through; reads of the stage take it as an input.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t &token) {
  for (uint32_t i = 0; i < ST_SPIN_LIMIT; i++)
    if ((token = mbar_try_wait(bar, parity)) != 0) return true;
  atomicExch(&g_stream_error, 1);
  return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// Shared-memory reads by 32-bit shared address (no generic-to-shared conversion per load).
// Each takes `token`, a value the compiler cannot see through, produced by the stage's barrier
// wait: reads of two different stages cannot be merged, and no read moves above the wait (nor,
// for x and the table, above the block-wide barrier that publishes them, which precedes it).
template <int OFF>
__device__ __forceinline__ uint32_t ring_u32(uint32_t addr, uint32_t token) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF), "r"(token));
  return v;
}
template <int OFF>
__device__ __forceinline__ uint32_t ring_u16(uint32_t addr, uint32_t token) {
  uint16_t v;
  asm("ld.shared.u16 %0, [%1+%2];" : "=h"(v) : "r"(addr), "n"(OFF), "r"(token));
  return v;
}
__device__ __forceinline__ uint32_t lut_read(uint32_t addr, uint32_t token) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr), "r"(token));
  return v;
}
template <int OFF>
__device__ __forceinline__ uint2 x_read(uint32_t addr, uint32_t token) {
  uint2 v;
  asm("ld.shared.v2.u32 {%0, %1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(OFF), "r"(token));
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

struct StreamArgs {
  bn_r4 w;
  const uint16_t *x;
  uint16_t *y;
  int64_t N, K;
  int T;
  int m;                       // input rows really present (<= M of the instantiation)
  int64_t x_stride, y_stride;  // elements between input rows / output rows (m > 1)
  int stages;                  // ring depth per warp
  uint32_t smem;  // dynamic shared memory of the launch, bytes
  // expert gather (blockIdx.y = slot g): rows ei[g] * RS + R0 .. + N, input row xi[g]; outputs
  // y [G, N], or with 0 < split < N: y [G, split] and y2 [G, N - split]. ei == nullptr: plain.
  const uint32_t *xi, *ei;
  int64_t RS, R0, split;
  uint16_t *y2;
  // grouped expert gather (M > 1, seg != nullptr): blockIdx.y = expert * chunks + chunk; the
  // expert's slots are order[seg[e] .. seg[e+1]) (slot numbers sorted by expert), this block
  // multiplies slots 8 * chunk .. of them (up to M): inputs x[xi[slot]], outputs row `slot`
  const uint32_t *seg, *order;
  int chunks;
};

// Where everything sits in the shared window, by absolute shared address (base = start of the
// dynamic allocation): [base, 64K) and [128K, end) hold the mbarriers and the per-warp rings,
// [64K, 128K) the pair table. An entry of the table is 256 bytes of which the lanes use the first
// 128: with one input row, x lives in the other halves (tile t's 256 bytes in the halves of
// entries 2t and 2t + 1, so a lane's address still grows by a constant per tile: 512 bytes, and
// K <= 16384); with several input rows, x sits above the table.
struct StreamLayout {
  uint32_t x_at, bar_at, tab_at, pool_a, pool_c, in_a, end;
};
__host__ __device__ inline StreamLayout stream_layout(uint32_t base, int T, int M, int warps, int S, uint32_t stage) {
  StreamLayout L;
  const uint32_t a0 = (base + 15u) & ~15u, xbytes = (uint32_t)M * (uint32_t)T * 256u, ring = (uint32_t)S * stage;
  if (M == 1) {
    L.x_at = 65536u + 128u, L.bar_at = a0, L.pool_c = 131072u;  // x in the unused halves of the table's entries
  } else {
    L.bar_at = a0, L.x_at = 131072u, L.pool_c = (131072u + xbytes + 127u) & ~127u;
  }
  L.tab_at = (L.bar_at + (uint32_t)warps * S * 8u + 15u) & ~15u;  // 16 exponent words while the table is built
  L.pool_a = (L.tab_at + 64u + 127u) & ~127u;
  L.in_a = L.pool_a < 65536u ? (65536u - L.pool_a) / ring : 0u;  // warps whose rings sit below the table
  if (L.in_a > (uint32_t)warps) L.in_a = warps;
  L.end = L.pool_c + ((uint32_t)warps - L.in_a) * ring;
  if (L.pool_a > 65536u) L.end = 0xFFFFFFFFu;  // x or the barriers would run into the table
  return L;
}

// Escapes of one flagged lane word, in weight order across the warp: exponent bits of its
// code-15 weights are OR-ed into the two BF16x2 words from the row's escape cursor, which then
// moves on by the tile's escape count. Nearly every flagged tile holds its escapes in a single
// lane: that lane reads them straight from the cursor and one shuffle tells the warp the count;
// the general case (several lanes) is a ballot scan kept out of line. Whole warp calls it.
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

// Bytes from one tile's x to the next in shared memory (see StreamLayout).
template <int M>
constexpr uint32_t X_TILE = M == 1 ? 512u : 256u;

// The M input rows' four BF16 values of one tile for this lane: row m sits `xrow` bytes after
// row m-1 in shared memory.
template <int M, int OFF>
__device__ __forceinline__ void x_tile(uint32_t xs, uint32_t xrow, uint32_t token, uint2 (&xv)[M]) {
#pragma unroll
  for (int m = 0; m < M; m++) xv[m] = x_read<OFF>(xs + m * xrow, token);
}

// Decode of lane word (row I, tile U) of a block, all offsets immediate, and its M products.
template <int I, int U, int M, uint32_t RAW_ROW, uint32_t CODE_ROW>
__device__ __forceinline__ void word_fma(uint32_t raw, uint32_t codes, uint32_t lut, uint32_t token, const uint2 (&xv)[M], float (&acc)[M]) {
  const uint32_t r4 = ring_u32<I * RAW_ROW + U * 128>(raw, token);
  const uint32_t c4 = ring_u16<I * CODE_ROW + U * 64>(codes, token);
  const uint32_t e01 = lut_read(__byte_perm(c4, lut, 0x7604), token);  // lut + code byte 0 * 256
  const uint32_t e23 = lut_read(__byte_perm(c4, lut, 0x7614), token);  // lut + code byte 1 * 256
  const uint32_t w01 = (__byte_perm(r4, 0u, 0x1100) & 0x807F807Fu) | e01;
  const uint32_t w23 = (__byte_perm(r4, 0u, 0x3322) & 0x807F807Fu) | e23;
#pragma unroll
  for (int m = 0; m < M; m++) acc[m] = fma2_bf16(w23, xv[m].y, fma2_bf16(w01, xv[m].x, acc[m]));
}

// NT tiles x RWG rows, straight-line: no loop, no test, every offset an immediate.
template <int RWG, int NT, int M, uint32_t RAW_ROW, uint32_t CODE_ROW, int U = 0>
__device__ __forceinline__ void block_fma(uint32_t raw, uint32_t codes, uint32_t xs, uint32_t xrow, uint32_t lut, uint32_t token, float (&acc)[RWG][M]) {
  if constexpr (U < NT) {
    uint2 xv[M];
    x_tile<M, U * X_TILE<M>>(xs, xrow, token, xv);
    word_fma<0, U, M, RAW_ROW, CODE_ROW>(raw, codes, lut, token, xv, acc[0]);
    if constexpr (RWG > 1) word_fma<1, U, M, RAW_ROW, CODE_ROW>(raw, codes, lut, token, xv, acc[1]);
    if constexpr (RWG > 2) word_fma<2, U, M, RAW_ROW, CODE_ROW>(raw, codes, lut, token, xv, acc[2]);
    if constexpr (RWG > 3) word_fma<3, U, M, RAW_ROW, CODE_ROW>(raw, codes, lut, token, xv, acc[3]);
    block_fma<RWG, NT, M, RAW_ROW, CODE_ROW, U + 1>(raw, codes, xs, xrow, lut, token, acc);
  }
}

// One tile of RWG rows with every check: escapes where fbits says so, lanes outside a partial
// tile masked. `u`: the tile's bit in fbits.
template <int RWG, int M, uint32_t RAW_ROW, uint32_t CODE_ROW, int I = 0>
__device__ __forceinline__ void careful_tile(uint32_t raw, uint32_t codes, uint32_t lut, uint32_t token, const uint2 (&xv)[M], int u, bool in, const uint32_t (&fbits)[RWG], const uint8_t *__restrict__ esc, uint32_t (&epos)[RWG], float (&acc)[RWG][M]) {
  if constexpr (I < RWG) {
    const uint32_t r4 = ring_u32<I * RAW_ROW>(raw, token);
    const uint32_t c4 = ring_u16<I * CODE_ROW>(codes, token);
    uint32_t w01 = (__byte_perm(r4, 0u, 0x1100) & 0x807F807Fu) | lut_read(__byte_perm(c4, lut, 0x7604), token);
    uint32_t w23 = (__byte_perm(r4, 0u, 0x3322) & 0x807F807Fu) | lut_read(__byte_perm(c4, lut, 0x7614), token);
    if ((fbits[I] >> u) & 1u) escape_patch(c4, esc, epos[I], w01, w23);
#pragma unroll
    for (int m = 0; m < M; m++) {
      const float s = fma2_bf16(w23, xv[m].y, fma2_bf16(w01, xv[m].x, acc[I][m]));
      acc[I][m] = in ? s : acc[I][m];
    }
    careful_tile<RWG, M, RAW_ROW, CODE_ROW, I + 1>(raw, codes, lut, token, xv, u, in, fbits, esc, epos, acc);
  }
}

// One stage (nt tiles) of RWG rows against M input rows, in blocks of BT tiles. A full block
// without a flagged tile (and not holding a row's partial last tile) runs as one straight line of
// code: no loop, no test, every offset an immediate. Any other block goes tile by tile with every
// check.
//   fbits[i]  bit u: tile u of row i holds escapes
//   partial   the stage's last tile is a row's partial last tile; lanes without
//             `lane_in_partial` hold no weight in it
template <int RWG, int KC, int M, uint32_t RAW_ROW, uint32_t CODE_ROW>
__device__ __forceinline__ void consume_stage(uint32_t raw, uint32_t codes, uint32_t xs, uint32_t xrow, uint32_t lut, uint32_t token, int nt, bool partial, bool lane_in_partial, const uint32_t (&fbits)[RWG], const uint8_t *__restrict__ esc, uint32_t (&epos)[RWG], float (&acc)[RWG][M]) {
  constexpr int BT = KC < 4 ? KC : (RWG * M >= 4 ? 2 : 4);
  constexpr int NB = (KC + BT - 1) / BT;
  uint32_t any = 0;
#pragma unroll
  for (int i = 0; i < RWG; i++) any |= fbits[i];
#pragma unroll
  for (int b = 0; b < NB; b++) {
    const int left = nt - b * BT;
    if (left <= 0) break;
    const uint32_t braw = raw + b * BT * 128, bcodes = codes + b * BT * 64, bxs = xs + b * BT * X_TILE<M>;
    const bool tail = partial && left <= BT;  // this block holds the partial tile
    if (left >= BT && !tail && !((any >> (b * BT)) & ((1u << BT) - 1u))) {
      block_fma<RWG, BT, M, RAW_ROW, CODE_ROW>(braw, bcodes, bxs, xrow, lut, token, acc);
    } else {
      const int n = left < BT ? left : BT;
      for (int k = 0; k < n; k++) {
        const bool in = lane_in_partial || !(tail && k == n - 1);
        uint2 xv[M];
        x_tile<M, 0>(bxs + k * X_TILE<M>, xrow, token, xv);
        careful_tile<RWG, M, RAW_ROW, CODE_ROW>(braw + k * 128, bcodes + k * 64, lut, token, xv, b * BT + k, in, fbits, esc, epos, acc);
      }
    }
  }
}

// WARPS: streaming warps per block (one block per SM); RW: rows walked together (a warp's last
// rows % RW rows are walked one at a time); KC: tiles per stage.
//
// Shared window, by absolute shared address (base = start of the dynamic allocation):
//   [base, 64K)    (x as BF16 [T*128] when M == 1) | mbarriers | rings of the first warps
//   [64K, 128K)    pair table
//   [128K, end)    (x [M][T*128] when M > 1) | rings of the remaining warps
// M: input rows multiplied in one pass (accumulators per weight row); rows >= a.m are zeros.
template <int WARPS, int RW, int KC, int M>
__global__ void __launch_bounds__(WARPS * 32, 1) r4_stream_kernel(StreamArgs a) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  static_assert(32 % KC == 0, "a stage must not straddle a 32-tile flag word");
  constexpr int THREADS = WARPS * 32;
  constexpr uint32_t RAW_ROW = KC * 128, CODE_ROW = KC * 64;
  constexpr uint32_t RAW_STAGE = RW * RAW_ROW, STAGE = RAW_STAGE + RW * CODE_ROW;
  constexpr uint32_t STAGE_MASK = (1u << KC) - 1u;
  const uint32_t lane = lane_id(), warp = threadIdx.x >> 5;
  const int64_t K = a.K;
  const int T = a.T, S = a.stages;
  const uint32_t base = smem_addr(smem_raw);
  const StreamLayout L = stream_layout(base, T, M, WARPS, S, STAGE);
  const uint32_t x_at = L.x_at, bar_at = L.bar_at, xrow = (uint32_t)T * 256u;
  const uint32_t s_ring = warp < L.in_a ? L.pool_a + warp * (uint32_t)S * STAGE : L.pool_c + (warp - L.in_a) * (uint32_t)S * STAGE;
  if (base > ST_BASE_MAX || L.end > base + a.smem) {  // the host sized the window for another layout
    if (threadIdx.x == 0) atomicExch(&g_stream_error, 2);
    return;
  }
  const uint32_t s_bar = bar_at + warp * (uint32_t)S * 8u;

  // this warp's rows: nfull groups of RW rows, then the remaining rows one per group
  // output rows of this warp: an even split of N over all warps of the grid (32-bit arithmetic
  // when it fits: a 64-bit division is a few hundred dependent instructions at kernel start)
  const uint32_t workers = gridDim.x * WARPS, me = blockIdx.x * WARPS + warp;
  int64_t o_begin, o_end;
  if ((uint64_t)a.N * workers < (1ull << 32)) {
    const uint32_t n32 = (uint32_t)a.N;
    o_begin = n32 * me / workers, o_end = n32 * (me + 1u) / workers;
  } else {
    o_begin = a.N * (int64_t)me / workers, o_end = a.N * (int64_t)(me + 1u) / workers;
  }
  const int64_t slot = blockIdx.y;
  if (!a.seg && a.ei && a.ei[slot] == BN_NO_EXPERT) return;  // a padding slot (whole block, before any barrier is armed)
  // grouped gather: this block's expert, its first slot in `order` and how many slots it takes
  int64_t g_first = 0;
  int g_count = a.m;
  if (a.seg) {
    const int64_t e = slot / a.chunks, c = slot % a.chunks;
    g_first = (int64_t)a.seg[e] + c * M;
    g_count = (int)max((int64_t)0, min((int64_t)M, (int64_t)a.seg[e + 1] - g_first));
    if (g_count == 0) return;  // whole block: nothing routed here
  }
  const int64_t row0 = a.seg ? (slot / a.chunks) * a.RS + a.R0 : a.ei ? (int64_t)a.ei[slot] * a.RS + a.R0 : 0;  // storage row of output row 0
  const int64_t r_begin = row0 + o_begin;
  const int nrows = (int)(o_end - o_begin);
  const int nfull = nrows / RW, ngroups = nfull + (nrows - nfull * RW);
  const int nchunks = (T + KC - 1) / KC, last_chunk = nchunks - 1;
  const int nt_last = T - last_chunk * KC;  // tiles of a row's last stage
  auto group_row = [&](int g) { return g < nfull ? g * RW : nfull * RW + (g - nfull); };

  if (lane == 0)
    for (int s = 0; s < S; s++) mbar_init(s_bar + s * 8, 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  __syncwarp();

  // Producer side. Lanes 0..RW-1 copy the raw bytes of rows 0..RW-1 of a group, lanes 16..16+RW-1
  // their code words. A lane's source pointer simply runs on through its row; at the end of a
  // group of RW rows it skips the rows its neighbours copied.
  const bool raw_lane = lane < 16;
  const uint32_t my_row = lane & 15u;
  const uint32_t my_step = raw_lane ? RAW_ROW : CODE_ROW;
  const uint32_t my_last = raw_lane ? (uint32_t)(K - (int64_t)last_chunk * KC * BN_TILE) : (uint32_t)nt_last * 64u;
  const uint32_t my_off = raw_lane ? my_row * RAW_ROW : RAW_STAGE + my_row * CODE_ROW;
  const uint32_t row_bytes = raw_lane ? (uint32_t)K : (uint32_t)T * 64u;
  const uint32_t tx_full = RAW_ROW + CODE_ROW;
  const uint32_t tx_last = (uint32_t)(K - (int64_t)last_chunk * KC * BN_TILE) + (uint32_t)nt_last * 64u;
  int pg = 0, pc = 0, ps = 0;
  const uint8_t *src = (raw_lane ? a.w.raw : reinterpret_cast<const uint8_t *>(a.w.codes)) + (r_begin + (int64_t)min(my_row, (uint32_t)max(nrows - 1, 0))) * row_bytes;
  auto issue = [&]() {
    if (pg >= ngroups) return;
    const bool last = pc == last_chunk, wide_g = pg < nfull;
    const uint32_t bytes = last ? my_last : my_step;
    const uint32_t bar = s_bar + (uint32_t)ps * 8u;
    if (lane == 0) mbar_expect_tx(bar, (last ? tx_last : tx_full) * (wide_g ? RW : 1));
    if (my_row < (wide_g ? (uint32_t)RW : 1u)) bulk_g2s(s_ring + (uint32_t)ps * STAGE + my_off, src, bytes, bar);
    src += bytes;
    if (last) {
      pc = 0, pg++;
      if (wide_g) src += (size_t)(RW - 1) * row_bytes;
    } else {
      pc++;
    }
    ps = ps + 1 == S ? 0 : ps + 1;
  };
  // flag bytes (one 32-tile group per row at a time) and escape cursors are fetched one step
  // ahead of their use, so their global-memory latency hides behind the previous tiles
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

  // Start-up order matters: the first ring fills ask for megabytes at once across the GPU, and a
  // load issued after them queues behind them. So the small loads everything waits on (x, the
  // table, the first rows' flags and cursors) are issued first, then the ring fills; their
  // results are consumed only afterwards.
  const int x_words = M * T * 16;  // 16-byte pieces of x
  auto x_piece = [&](int i) {
    const int m = i / (T * 16), j = i - m * (T * 16);
    if (m >= g_count || (int64_t)j * 8 >= K) return make_uint4(0, 0, 0, 0);  // K % 16 == 0
    const int64_t xrow = a.seg ? (int64_t)a.xi[a.order[g_first + m]] : a.ei ? (int64_t)a.xi[slot] : -1;
    const uint4 *x8 = reinterpret_cast<const uint4 *>(a.x + (xrow >= 0 ? xrow * K : (int64_t)m * a.x_stride));
    return __ldg(x8 + j);
  };
  const uint32_t tab_byte = threadIdx.x < 15 ? (uint32_t)__ldg(a.w.table + threadIdx.x) : 0u;
  const uint4 x_first = (int)threadIdx.x < x_words ? x_piece(threadIdx.x) : make_uint4(0, 0, 0, 0);
  if (ngroups > 0) prefetch_flags(0, 0), prefetch_epos(0);
  for (int s = 0; s < S; s++) issue();

  // x and the pair table into shared memory (whole block). The 15 table bytes go through shared
  // memory first, so the 8192 table words are built from on-chip reads.
  {
    uint32_t *s_tab = reinterpret_cast<uint32_t *>(smem_raw + (L.tab_at - base));
    if (threadIdx.x < 16) s_tab[threadIdx.x] = tab_byte;
    // 16-byte piece i of x: input row i / (T * 16), piece j of that row = bytes 16 j .. of it
    auto x_dst = [&](int i) {
      if (M > 1) return reinterpret_cast<uint4 *>(smem_raw + (x_at - base)) + i;
      const uint32_t t = (uint32_t)i >> 4, p = (uint32_t)i & 15u;  // tile, piece of the tile
      return reinterpret_cast<uint4 *>(smem_raw + (x_at - base) + (2u * t + (p >> 3)) * 256u + (p & 7u) * 16u);
    };
    if ((int)threadIdx.x < x_words) *x_dst(threadIdx.x) = x_first;
    for (int i = threadIdx.x + THREADS; i < x_words; i += THREADS) *x_dst(i) = x_piece(i);
    __syncthreads();
    uint32_t *lut = reinterpret_cast<uint32_t *>(smem_raw + (65536u - base));
#pragma unroll 4
    for (uint32_t i = threadIdx.x; i < 256 * 32; i += THREADS) {
      const uint32_t code = i >> 5, l = i & 31;
      lut[code * 64 + l] = (s_tab[code & 15] << 7) | (s_tab[code >> 4] << 23);  // entry 15: no exponent bits
    }
    __syncthreads();
  }

  const uint32_t lut_lane = 65536u + lane * 4;
  // in a row's partial last tile (K % 128 != 0) only the lanes below K % 128 hold weights
  const bool has_partial = (K & 127) != 0;
  const bool lane_in_partial = (int64_t)lane * 4 < (K & 127);
  int cs = 0;           // consumer slot
  uint32_t phases = 0;  // bit s: parity to wait for on slot s
  const int fgroups = (T + 31) / 32;
  for (int g = 0; g < ngroups; g++) {
    const bool wide = g < nfull;
    const int64_t row = r_begin + group_row(g);
    float acc[RW][M];
    uint32_t epos[RW], fmask[RW];
#pragma unroll
    for (int i = 0; i < RW; i++) {
      epos[i] = pf_epos[i], fmask[i] = 0u;
#pragma unroll
      for (int m = 0; m < M; m++) acc[i][m] = 0.0f;
    }
    if (g + 1 < ngroups) prefetch_epos(g + 1);
    uint32_t xs = M == 1 ? x_at + (lane >> 4) * 256u + (lane & 15u) * 8u : x_at + lane * 8u;
    for (int c = 0; c < nchunks; c++) {
      const int t0 = c * KC;
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
      uint32_t token;
      if (!mbar_wait(s_bar + (uint32_t)cs * 8, (phases >> cs) & 1u, token)) return;  // gave up: status flag is set
      phases ^= 1u << cs;
      const uint32_t raw = s_ring + (uint32_t)cs * STAGE + lane * 4;
      const uint32_t codes = s_ring + (uint32_t)cs * STAGE + RAW_STAGE + lane * 2;
      const bool last = c == last_chunk;
      const int nt = last ? nt_last : KC;
      const bool partial = last && has_partial;
      if (wide) {
        uint32_t fbits[RW];
#pragma unroll
        for (int i = 0; i < RW; i++) fbits[i] = (fmask[i] >> (t0 & 31)) & STAGE_MASK;
        consume_stage<RW, KC, M, RAW_ROW, CODE_ROW>(raw, codes, xs, xrow, lut_lane, token, nt, partial, lane_in_partial, fbits, a.w.esc, epos, acc);
      } else {
        uint32_t fb1[1] = {(fmask[0] >> (t0 & 31)) & STAGE_MASK}, ep1[1] = {epos[0]};
        float ac1[1][M];
#pragma unroll
        for (int m = 0; m < M; m++) ac1[0][m] = acc[0][m];
        consume_stage<1, KC, M, RAW_ROW, CODE_ROW>(raw, codes, xs, xrow, lut_lane, token, nt, partial, lane_in_partial, fb1, a.w.esc, ep1, ac1);
        epos[0] = ep1[0];
#pragma unroll
        for (int m = 0; m < M; m++) acc[0][m] = ac1[0][m];
      }
      xs += KC * X_TILE<M>;
      // every read of the slot feeds an accumulator: pin them before the slot is refilled
#pragma unroll
      for (int i = 0; i < RW; i++)
#pragma unroll
        for (int m = 0; m < M; m++) asm volatile("" ::"f"(acc[i][m]) : "memory");
      __syncwarp();
      issue();  // refill the slot just drained
      cs = cs + 1 == S ? 0 : cs + 1;
    }
    // lane i * M + m ends up with the sum of (row i, input m)
    float mine = 0.0f;
#pragma unroll
    for (int i = 0; i < RW; i++)
#pragma unroll
      for (int m = 0; m < M; m++) {
        float s = acc[i][m];
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) s = s + __shfl_xor_sync(BN_FULL, s, o);
        if ((int)lane == i * M + m) mine = s;
      }
    const int li = (int)lane / M, lm = (int)lane % M;  // this lane's (row, input)
    if (li < (wide ? RW : 1) && lm < g_count) {
      const int64_t r = row - row0 + li;  // output row within the slot
      const uint16_t v = f32_to_bf16_bits(mine);
      if (a.seg) {
        const int64_t o = a.order[g_first + lm];  // the slot this input row belongs to
        if (a.split > 0 && r >= a.split) a.y2[o * (a.N - a.split) + (r - a.split)] = v;
        else a.y[o * (a.split > 0 ? a.split : a.N) + r] = v;
      } else if (M > 1) a.y[(int64_t)lm * a.y_stride + r] = v;
      else if (a.split > 0 && r >= a.split) a.y2[slot * (a.N - a.split) + (r - a.split)] = v;
      else a.y[slot * (a.split > 0 ? a.split : a.N) + r] = v;
    }
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

constexpr uint32_t ST_SMEM_MAX = 227 * 1024;  // dynamic shared memory one block may ask for

// Ring depth that fits the shared window when the dynamic allocation starts at `base` (the
// kernel's own layout arithmetic); 0 if not even two stages per warp fit.
static int stream_stages(int warps, uint32_t stage, int T, int M, uint32_t base) {
  for (int S = 6; S >= 2; S--)
    if (stream_layout(base, T, M, warps, S, stage).end <= ST_SMEM_MAX) return S;  // the window ends at base + ST_SMEM_MAX >= ST_SMEM_MAX
  return 0;
}

template <int WARPS, int RW, int KC, int M = 1>
static int launch_stream(StreamArgs a, cudaStream_t s, int64_t slots = 1, int64_t active = 0) {
  // worst case of the two extremes of the window's start; the kernel re-derives the layout
  // from the real start and refuses to run if it does not fit
  const int stages = min(stream_stages(WARPS, RW * KC * 192, a.T, M, 0), stream_stages(WARPS, RW * KC * 192, a.T, M, ST_BASE_MAX));
  if (stages < 2) return -1;  // does not fit: caller falls back
  a.stages = stages;
  a.smem = ST_SMEM_MAX;
  if (a.m < 1) a.m = 1;
  auto kern = r4_stream_kernel<WARPS, RW, KC, M>;
  BN_CUDA(allow_smem(kern, a.smem));
  if (active < 1 || active > slots) active = slots;  // slots expected to have work (a grouped gather leaves many empty)
  int64_t blocks = (stream_sms() + active - 1) / active;  // blocks per slot: about one block per SM in all
  const int64_t need = (a.N + WARPS - 1) / WARPS;
  if (blocks > need) blocks = need;
  kern<<<dim3((unsigned)blocks, (unsigned)slots), WARPS * 32, a.smem, s>>>(a);
  return launched("r4_stream_kernel");
}

// Returns -1 when the shape is outside what the streaming kernel covers. More resident warps
// hide more of the decode's dependent-issue latency, so the widest block whose rings still fit
// the shared window next to x is taken (24 warps for K = 3840, 20 for K = 15360).
// The bulk copies and the 16-byte reads of x need 16-byte aligned arrays.
static bool stream_aligned(const bn_r4 *w, const uint16_t *x) {
  return ((reinterpret_cast<uintptr_t>(w->raw) | reinterpret_cast<uintptr_t>(w->codes) | reinterpret_cast<uintptr_t>(x)) & 15) == 0;
}

int stream_matvec(const bn_r4 *w, const uint16_t *x, int64_t N, int64_t K, uint16_t *y, cudaStream_t s) {
  const int64_t T = tiles(K);
  if (K % 16 || N < 1 || T > 128 || !stream_aligned(w, x)) return -1;  // x lives in the table's 256 half entries, two per tile
  StreamArgs a{};
  a.w = *w, a.x = x, a.y = y, a.N = N, a.K = K, a.T = (int)T;
  // 26 warps when that evens the rows out (15360 rows over 148 SMs: 104 per SM = 26 x 4, against
  // 4 or 5 per warp with 24), else the widest block whose rings fit
  const int64_t per_sm = (N + stream_sms() - 1) / stream_sms();
  int e = -1;
  if ((per_sm + 25) / 26 < (per_sm + 23) / 24) e = launch_stream<26, 2, 8>(a, s);
  if (e == -1) e = launch_stream<24, 2, 8>(a, s);
  if (e == -1) e = launch_stream<20, 2, 8>(a, s);
  if (e == -1) e = launch_stream<16, 2, 8>(a, s);
  if (e == -1) e = launch_stream<8, 2, 8>(a, s);
  return e;
}

// Expert gather through the streaming kernel; -1 when the shape is outside its coverage.
int stream_gather(const bn_r4 *w, const uint16_t *x, const uint32_t *xi, const uint32_t *ei, int64_t G, int64_t n, int64_t K, int64_t RS, int64_t R0, int64_t split, uint16_t *y, uint16_t *y2, cudaStream_t s) {
  const int64_t T = tiles(K);
  if (K % 16 || n < 1 || T > 128 || G < 1 || G > 65535 || !stream_aligned(w, x)) return -1;
  StreamArgs a{};
  a.w = *w, a.x = x, a.y = y, a.y2 = y2, a.N = n, a.K = K, a.T = (int)T;
  a.xi = xi, a.ei = ei, a.RS = RS, a.R0 = R0, a.split = split;
  int e = launch_stream<24, 2, 8>(a, s, G);
  if (e == -1) e = launch_stream<20, 2, 8>(a, s, G);
  if (e == -1) e = launch_stream<16, 2, 8>(a, s, G);
  if (e == -1) e = launch_stream<8, 2, 8>(a, s, G);
  return e;
}

// Grouped expert gather: every expert's slots in blocks of M input rows; -1 outside coverage.
template <int M>
static int stream_grouped_m(StreamArgs a, cudaStream_t s, int64_t groups, int64_t active) {
  int e = launch_stream<16, 2, 8, M>(a, s, groups, active);
  if (e == -1) e = launch_stream<12, 2, 8, M>(a, s, groups, active);
  if (e == -1) e = launch_stream<8, 2, 8, M>(a, s, groups, active);
  return e;
}

int stream_gather_grouped(const bn_r4 *w, const uint16_t *x, const uint32_t *xi, const uint32_t *seg, const uint32_t *order, int64_t E, int64_t G, int64_t max_per_expert, int64_t n, int64_t K, int64_t RS, int64_t R0, int64_t split, uint16_t *y, uint16_t *y2, cudaStream_t s) {
  const int64_t T = tiles(K);
  if (K % 16 || n < 1 || T > 200 || E < 1 || max_per_expert < 1 || !stream_aligned(w, x)) return -1;
  const int m = max_per_expert <= 4 ? 4 : 8;
  const int64_t chunks = (max_per_expert + m - 1) / m;
  if (E * chunks > 65535) return -1;
  StreamArgs a{};
  a.w = *w, a.x = x, a.y = y, a.y2 = y2, a.N = n, a.K = K, a.T = (int)T, a.m = m;
  a.xi = xi, a.RS = RS, a.R0 = R0, a.split = split, a.seg = seg, a.order = order, a.chunks = (int)chunks;
  const int64_t active = G < E ? G : E;  // experts with work: at most one per slot
  return m == 4 ? stream_grouped_m<4>(a, s, E * chunks, active) : stream_grouped_m<8>(a, s, E * chunks, active);
}

// 2..8 input rows through the streaming kernel (weights stream once, M accumulators per weight
// row, every output in the documented order); -1 when the shape is outside its coverage.
template <int M>
static int stream_rows_m(StreamArgs a, cudaStream_t s) {
  int e = launch_stream<16, 2, 8, M>(a, s);
  if (e == -1) e = launch_stream<12, 2, 8, M>(a, s);
  if (e == -1) e = launch_stream<8, 2, 8, M>(a, s);
  return e;
}

int stream_rows(const bn_r4 *w, const uint16_t *x, int64_t x_stride, int64_t M, int64_t N, int64_t K, uint16_t *y, int64_t y_stride, cudaStream_t s) {
  const int64_t T = tiles(K);
  if (K % 16 || x_stride % 8 || N < 1 || T > 200 || M < 2 || M > 8 || !stream_aligned(w, x)) return -1;
  StreamArgs a{};
  a.w = *w, a.x = x, a.y = y, a.N = N, a.K = K, a.T = (int)T;
  a.m = (int)M, a.x_stride = x_stride, a.y_stride = y_stride;
  if (M == 2) return stream_rows_m<2>(a, s);
  if (M <= 4) return stream_rows_m<4>(a, s);
  return stream_rows_m<8>(a, s);
}

int stream_status_reset() {
  const int zero = 0;
  BN_CUDA(cudaMemcpyToSymbol(g_stream_error, &zero, sizeof(int)));
  return BN_OK;
}

}  // namespace bn

extern "C" int bn_device_status_reset(void) {
  if (int e = bn::stream_status_reset()) return e;
  if (int e = bn::oct_status_reset()) return e;
  if (int e = bn::mma_status_reset()) return e;
  return bn::exchange_status_reset();
}

extern "C" int bn_device_status(int *status) {
  if (!status) return bn::fail(BN_ERR_ARG, "bn_device_status: null pointer");
  int stream = 0, mma = 0, xch = 0, oct = 0;
  BN_CUDA(cudaMemcpyFromSymbol(&stream, bn::g_stream_error, sizeof(int)));
  if (int e = bn::oct_status(&oct)) return e;
  if (oct) stream |= 4;
  if (int e = bn::mma_status(&mma)) return e;
  if (int e = bn::exchange_status(&xch)) return e;
  *status = stream | (mma << 8) | (xch << 16);
  return BN_OK;
}
