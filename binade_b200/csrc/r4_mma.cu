// Fused R4-decode GEMM for up to 256 input rows on the 5th-generation tensor cores (tcgen05):
//   Y[m, n] = sum_k X[m, k] W[n, k]      X [M, K] BF16, W [N, K] in R4, Y [M, N] BF16
// computed as D = W_tile . X^T so that the few input rows sit in the MMA's N dimension:
//   A operand  a block's weight rows x 128 k, decoded from R4 to BF16 by the CUDA cores straight
//              into shared memory in the tensor core's K-major 128-byte-swizzled layout
//   B operand  BN = M rounded up to 16 input rows x 128 k, brought in by TMA (2-D tensor map over
//              X with the same swizzle; rows past M and columns past K arrive as zeros)
//   D          128 x BN fp32 accumulators in tensor memory (TMEM), read back with tcgen05.ld
// One block per SM, each with an equal share of the weight rows; one warp issues the TMA copies
// and the MMAs; a ring of stages (mbarriers: `full` armed by the decoders and the TMA bytes,
// `empty` by tcgen05.commit) lets decode run ahead. Two decode sides:
//   r4_mma_oct_kernel  up to 128 input rows, K % 16 == 0: 26 warps, eight threads per weight row,
//                      private cp.async rings (the batch-1 matvec's decode, oct.cuh)
//   r4_mma_kernel      the rest: 14 warps, a warp per row and stage, 8 rows each, raw bytes and
//                      codes fetched two stages ahead into registers
// The weights are read once whatever M. The sum over K is the hardware's: 16 k per MMA step, in
// order, from zero, in fp32: not the documented lane order of the one-row kernels, but the
// order of cuBLAS's BF16 GEMM on this GPU, whose outputs this kernel reproduces bit for bit;
// where cuBLAS splits K, `split` slices are summed in accumulators of their own and added in
// slice order by the epilogue (bn_r4_mma_split).
//
// Every wait is bounded: when one gives up, a status flag is set, every thread still reaches the
// end of the kernel, and the tensor memory is released.
#include <cuda.h>
#include <stdio.h>
#include <stdlib.h>

#include "common.cuh"
#include "decode.cuh"
#include "oct.cuh"

namespace bn {

constexpr int MMA_DECODE_WARPS = 14;  // decode warps of the shape used (measured: 14 x 8 rows 46 us, 28 x 4 rows 55 us on 15360 x 3840)
constexpr int MMA_RPW = 8;            // weight rows per decode warp and stage
constexpr int MMA_OCT_WARPS = 26;     // decode warps of the eight-threads-per-row kernel: 104 rows a block, 15360 rows in 148 blocks
constexpr int MMA_BM = 128;                  // MMA M: rows of the A tile (the block's rows, then unused)
constexpr int MMA_BK = 128;                  // k per stage: one R4 tile
constexpr uint32_t MMA_A_STAGE = MMA_BM * MMA_BK * 2;  // 32 KB: two 64-k atoms of 128 rows x 128 B
constexpr uint32_t MMA_SPIN_LIMIT = 1u << 22;
constexpr uint32_t MMA_SMEM_MAX = 226 * 1024;  // dynamic part; the pair-table builder keeps 64 static bytes

__device__ int g_mma_error;  // 1: a bounded wait gave up

__device__ __forceinline__ void mm_bar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mm_bar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mm_bar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ bool mm_bar_wait(uint32_t bar, uint32_t parity) {
  // (a try with a suspend-time hint compiles to a sleep-and-poll loop of its own: more
  // instructions for the same wait, measured, so the plain form is kept)
  for (uint32_t i = 0; i < MMA_SPIN_LIMIT; i++) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  atomicExch(&g_mma_error, 1);
  return false;
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major, 128-byte-swizzled operand tile that starts at
// shared address `addr` (1024-byte aligned atom; `addr` may point 32 * j bytes into the first
// row to select the j-th group of 16 k): start address >> 4 in bits 0..13, leading byte offset
// (unused for swizzled K-major, set to 1) in 16..29, stride between 8-row groups (1024 B) >> 4
// in 32..45, descriptor version 1 in 46..47, layout 2 = 128-byte swizzle in 61..63.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: fp32 accumulate (bits 4..5 = 1), A and B BF16 (bits 7..9, 10..12 = 1),
// both K-major (bits 15, 16 = 0), N >> 3 in bits 17..22, M >> 4 in bits 24..28.
__host__ __device__ constexpr uint32_t mma_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void mma_bf16(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

struct MmaArgs {
  bn_r4 w;
  uint16_t *y;
  int64_t N, K, y_stride;
  int T, M, BN, stages;
  int rows;  // weight rows per block (a multiple of MMA_RPW, at most MMA_ROWS)
  uint32_t tmem_cols;
  // split-K as cuBLAS does it for few input rows and long K: `split` equal slices of the K tiles,
  // each summed from zero into its own accumulator (BN columns apart in tensor memory), the
  // slices' fp32 sums added in slice order, then one rounding to BF16
  int split, slice_tiles;
};

// Byte offset of (row r, 16-byte chunk c of the row's 128 bytes) inside a swizzled atom.
__device__ __forceinline__ uint32_t swz(uint32_t r, uint32_t c) { return r * 128u + ((c ^ (r & 7u)) << 4); }

// Shared addresses of a block's stage ring and barriers.
struct MmaWindow {
  uint32_t a_at, b_at, b_stage;      // A stages, B stages, bytes of a B stage
  uint32_t full, empty, done, slot;  // full[S], empty[S], done, the word that receives the TMEM address
};

// The MMA warp: TMA copies of X and the MMAs of every k-tile. Returns false when a wait gave up.
__device__ __forceinline__ bool mma_issue_side(const CUtensorMap *x_map, const MmaWindow &m, int T, int S, int BN, int slice_tiles, uint32_t tmem, uint32_t lane, bool ok) {
  const uint32_t idesc = mma_idesc(MMA_BM, BN);
  auto fetch_x = [&](int t, int s) {  // X tile of k-tile t into slot s, which must be free
    const uint32_t b_s = m.b_at + (uint32_t)s * m.b_stage;
    mm_bar_expect_tx(m.full + 8 * s, m.b_stage);
    tma_load_2d(b_s, x_map, t * MMA_BK, 0, m.full + 8 * s);
    tma_load_2d(b_s + (uint32_t)BN * 128u, x_map, t * MMA_BK + 64, 0, m.full + 8 * s);
  };
  if (lane == 0)
    for (int t = 0; t < S && t < T; t++) fetch_x(t, t);
  __syncwarp();
  int s = 0, sp = 0;        // slot of tile t, slot of tile t - 1
  uint32_t ph = 0, php = 0;  // parity of their current phases
  int in_slice = 0;          // tile index inside the current K slice
  uint32_t acc = tmem;       // the slice's accumulator
  for (int t = 0; t < T; t++) {
    if (ok) ok = mm_bar_wait(m.full + 8 * s, ph);
    tc_fence_after();
    if (lane == 0 && ok) {
      const uint32_t a_s = m.a_at + (uint32_t)s * MMA_A_STAGE, b_s = m.b_at + (uint32_t)s * m.b_stage;
#pragma unroll
      for (int j = 0; j < MMA_BK / 16; j++) {  // 16 k per MMA: 32 bytes further along the swizzled row
        const uint64_t da = smem_desc(a_s + (j >> 2) * (MMA_BM * 128u) + (j & 3) * 32u);
        const uint64_t db = smem_desc(b_s + (j >> 2) * ((uint32_t)BN * 128u) + (j & 3) * 32u);
        mma_bf16(acc, da, db, idesc, (in_slice | j) != 0);
      }
      mma_commit(m.empty + 8 * s);  // arrives when these MMAs have read the stage
    }
    __syncwarp();
    // The slot of the previous tile takes the X tile that will use it next. Waiting for that
    // tile's MMAs here costs nothing (they were issued a whole stage ago), whereas waiting for
    // the MMAs just issued would put their latency between every two stages.
    if (t >= 1 && t - 1 + S < T) {
      if (ok) ok = mm_bar_wait(m.empty + 8 * sp, php);
      if (lane == 0 && ok) fetch_x(t - 1 + S, sp);
      __syncwarp();
    }
    sp = s, php = ph;
    if (++s == S) s = 0, ph ^= 1u;
    if (++in_slice == slice_tiles) in_slice = 0, acc += (uint32_t)BN;
  }
  if (lane == 0 && ok) mma_commit(m.done);
  __syncwarp();
  return ok;
}

// Warps 0..3: accumulators out of tensor memory (TMEM lane = weight row of the block), rounded to
// BF16 and stored.
__device__ __forceinline__ void mma_store_side(const MmaArgs &a, const MmaWindow &m, uint32_t tmem, uint32_t warp, uint32_t lane, int64_t row_base, int rows, bool ok) {
  if (ok) ok = mm_bar_wait(m.done, 0);
  tc_fence_after();
  const int r = (int)(warp * 32 + lane);
  if (!ok) return;
  if (a.split == 1) {  // the common case, kept free of the slice loop
    for (int c = 0; c < a.BN; c += 8) {
      uint32_t v[8];
      asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                   : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                   : "r"(tmem + ((warp * 32u) << 16) + (uint32_t)c));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int i = 0; i < 8; i++)
        if (c + i < a.M && r < rows) a.y[(int64_t)(c + i) * a.y_stride + row_base + r] = f32_to_bf16_bits(__uint_as_float(v[i]));
    }
    return;
  }
  for (int c = 0; c < a.BN; c += 8) {
    float sum[8];
    for (int sl = 0; sl < a.split; sl++) {  // the slices' sums, added in slice order
      uint32_t v[8];
      asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                   : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                   : "r"(tmem + ((warp * 32u) << 16) + (uint32_t)(sl * a.BN + c)));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int i = 0; i < 8; i++) sum[i] = sl ? sum[i] + __uint_as_float(v[i]) : __uint_as_float(v[i]);
    }
#pragma unroll
    for (int i = 0; i < 8; i++)
      if (c + i < a.M && r < rows) a.y[(int64_t)(c + i) * a.y_stride + row_base + r] = f32_to_bf16_bits(sum[i]);
  }
}

// DW decode warps (plus the MMA warp), RPW weight rows per decode warp and stage: a block takes
// up to DW * RPW <= 128 weight rows.
template <int DW, int RPWT>
__global__ void __launch_bounds__((DW + 1) * 32, 1) r4_mma_kernel(const __grid_constant__ CUtensorMap x_map, MmaArgs a) {
  constexpr int MMA_DECODE_WARPS = DW, MMA_RPW = RPWT;
  static_assert(DW * RPWT <= MMA_BM, "a block's rows are the MMA's M");
  extern __shared__ uint8_t mma_smem[];
  const uint32_t lane = lane_id(), warp = threadIdx.x >> 5, lt = lanemask_lt();
  const int T = a.T, S = a.stages, BN = a.BN;
  const int64_t K = a.K;
  const uint32_t b_stage = (uint32_t)BN * MMA_BK * 2u;  // two 64-k atoms of BN rows x 128 B
  // shared window: A stages | B stages | pair table | barriers
  const uint32_t base = (smem_addr(mma_smem) + 1023u) & ~1023u;
  const uint32_t a_at = base, b_at = a_at + (uint32_t)S * MMA_A_STAGE, lut_at = b_at + (uint32_t)S * b_stage;
  const uint32_t bar_at = lut_at + LUT_WORDS * 4u;  // full[S], empty[S], done, then the TMEM address
  const uint32_t full = bar_at, empty = bar_at + 8u * S, done = bar_at + 16u * S, slot = done + 8u;
  const MmaWindow win{a_at, b_at, b_stage, full, empty, done, slot};
  uint8_t *const gen = mma_smem + (base - smem_addr(mma_smem));  // generic pointer to `base`

  const int64_t row_base = (int64_t)blockIdx.x * a.rows;
  const int rows = (int)min((int64_t)a.rows, a.N - row_base);  // this block's weight rows
  const uint32_t active = (uint32_t)(rows + MMA_RPW - 1) / MMA_RPW;  // decode warps with rows

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; s++) mm_bar_init(full + 8 * s, active + 1), mm_bar_init(empty + 8 * s, 1);
    mm_bar_init(done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_DECODE_WARPS) {  // the MMA warp owns the tensor memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(a.tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  build_pair_lut(reinterpret_cast<uint32_t *>(gen + (lut_at - base)), a.w.table);  // syncs once inside
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem) : "r"(slot));

  bool ok = true;

  if (warp < active) {
    // ---------------------------------------------------------------- decode side
    constexpr int RPW = MMA_RPW;
    const uint32_t lut_lane = lut_at + lane * 4u;
    const uint32_t r0 = warp * RPW;
    // A warp slot past the block's last row decodes that last row again (its MMA row is never
    // stored), so the loop needs no per-row predicate. Row pointers are formed once.
    // (32-bit offsets from the block's first row: a block spans at most 112 rows.)
    uint32_t epos[RPW], a_off[RPW], raw_off[RPW], cod_off[RPW];
    const uint8_t *const raw_blk = a.w.raw + row_base * K;
    const uint16_t *const cod_blk = a.w.codes + row_base * T * 32;
    const uint8_t *const flag_blk = a.w.flags + row_base * T;
#pragma unroll
    for (int i = 0; i < RPW; i++) {
      const uint32_t r = (uint32_t)min((int)(r0 + i), rows - 1);
      epos[i] = a.w.row_esc[row_base + r];
      raw_off[i] = r * (uint32_t)K + lane * 4u;
      cod_off[i] = r * (uint32_t)T * 32u + lane;
      a_off[i] = (lane >> 4) * (MMA_BM * 128u) + (lane & 1u) * 8u + swz(r0 + i, (lane & 15u) >> 1);
    }
    const uint32_t flag_off = (uint32_t)min((int)(r0 + (lane < RPW ? lane : 0u)), rows - 1) * (uint32_t)T;
    // a row's last tile may be partial (K % 128 != 0): lanes past the row's end read nothing and
    // store zeros (the matching columns of X arrive as zeros, but 0 x Inf must not happen)
    const bool in_last = (int64_t)(T - 1) * BN_TILE + (int64_t)lane * 4 < K;
    auto load_stage = [&](int t, uint32_t (&rw)[RPW], uint32_t (&cd)[RPW], uint32_t &flag) {
      if (t < T) {
        const bool in = t < T - 1 || in_last;
#pragma unroll
        for (int i = 0; i < RPW; i++) {
          rw[i] = in ? ldg_stream_u32(raw_blk + (raw_off[i] + (uint32_t)t * BN_TILE)) : 0u;
          cd[i] = ldg_stream_u16(cod_blk + (cod_off[i] + (uint32_t)t * 32u));
        }
        flag = lane < RPW ? (uint32_t)flag_blk[flag_off + (uint32_t)t] : 0u;
      }
    };
    // raw bytes, codes and flags of the next two stages wait in registers
    uint32_t rw0[RPW] = {}, cd0[RPW] = {}, fl0 = 0, rw1[RPW] = {}, cd1[RPW] = {}, fl1 = 0;
    load_stage(0, rw0, cd0, fl0);
    load_stage(1, rw1, cd1, fl1);
    int s = 0;
    uint32_t ph = 1;  // parity of the `empty` phase that frees slot s (first pass: slots start free)
    for (int t = 0; t < T; t++) {
      uint32_t rw2[RPW] = {}, cd2[RPW] = {}, fl2 = 0;
      load_stage(t + 2, rw2, cd2, fl2);
      if (t >= S && ok) ok = mm_bar_wait(empty + 8 * s, ph);
      tc_fence_after();
      const uint32_t fmask = __ballot_sync(BN_FULL, fl0 != 0);
      const uint32_t a_s = a_at + (uint32_t)s * MMA_A_STAGE;
      const bool zero = t == T - 1 && !in_last;
#pragma unroll
      for (int i = 0; i < RPW; i++) {
        uint32_t w01, w23;
        decode4(rw0[i], cd0[i], lut_lane, w01, w23);
        if ((fmask >> i) & 1u) apply_escapes(cd0[i], a.w.esc, epos[i], lt, w01, w23);
        if (zero) w01 = 0u, w23 = 0u;
        asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(a_s + a_off[i]), "r"(w01), "r"(w23) : "memory");
      }
      fence_async_smem();  // the tensor core reads shared memory through the async proxy
      __syncwarp();
      if (lane == 0) mm_bar_arrive(full + 8 * s);
#pragma unroll
      for (int i = 0; i < RPW; i++) rw0[i] = rw1[i], cd0[i] = cd1[i], rw1[i] = rw2[i], cd1[i] = cd2[i];
      fl0 = fl1, fl1 = fl2;
      if (++s == S) s = 0, ph ^= 1u;
    }
  } else if (warp == MMA_DECODE_WARPS) {
    ok = mma_issue_side(&x_map, win, T, S, BN, a.slice_tiles, tmem, lane, ok);
  }
  if (warp < 4) mma_store_side(a, win, tmem, warp, lane, row_base, rows, ok);
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_DECODE_WARPS) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(a.tmem_cols) : "memory");
}

// The same GEMM with the decode side of the batch-1 matvec: eight threads per weight row (a thread
// decodes 16 consecutive weights of every tile: two 16-byte chunks of the swizzled A row), four
// rows per warp, up to 26 decode warps = 104 rows per block, every thread streaming its own bytes
// through a private cp.async ring of D tiles. About half the instructions per weight of the
// kernel above (one 16-byte and one 8-byte shared load bring what eight 4-byte and 2-byte global
// loads brought; the escape patch runs once per four rows), which is what bounds both. Takes
// M <= 128 (the rings need the shared memory that wider B stages would use) and K % 16 == 0.
template <int MAXW, int D, bool COLS>
__global__ void __launch_bounds__((MAXW + 1) * 32, 1) r4_mma_oct_kernel(const __grid_constant__ CUtensorMap x_map, MmaArgs a) {
  constexpr int R = 4;
  using Geo = OctGeom<R>;
  constexpr uint32_t SLOT = Geo::SLOT, RING = D * SLOT;
  extern __shared__ uint8_t mma_smem[];
  const uint32_t lane = lane_id(), warp = threadIdx.x >> 5;
  const int T = a.T, S = a.stages, BN = a.BN;
  const int64_t K = a.K;
  const uint32_t b_stage = (uint32_t)BN * MMA_BK * 2u;
  // shared window: A stages | B stages | pair table | barriers | rings
  const uint32_t base = (smem_addr(mma_smem) + 1023u) & ~1023u;
  const uint32_t a_at = base, b_at = a_at + (uint32_t)S * MMA_A_STAGE, lut_at = b_at + (uint32_t)S * b_stage;
  const uint32_t bar_at = lut_at + LUT_WORDS * 4u, ring_at = bar_at + 256u;
  const MmaWindow win{a_at, b_at, b_stage, bar_at, bar_at + 8u * S, bar_at + 16u * S, bar_at + 16u * S + 8u};
  uint8_t *const gen = mma_smem + (base - smem_addr(mma_smem));

  const int64_t row_base = (int64_t)blockIdx.x * a.rows;
  const int rows = (int)min((int64_t)a.rows, a.N - row_base);
  const uint32_t active = (uint32_t)(rows + R - 1) / R;  // decode warps with rows

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; s++) mm_bar_init(win.full + 8 * s, active + 1), mm_bar_init(win.empty + 8 * s, 1);
    mm_bar_init(win.done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MAXW) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(win.slot), "r"(a.tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }

  // ---- load side of a decode warp, started before the table is built
  const uint32_t grp = lane >> 3, p = lane & 7u;
  const uint32_t r = warp * R + grp;  // row of the A tile (and of the block)
  const int64_t srow = row_base + min((int)r, rows - 1);  // a slot past the block's last row decodes that row again; its MMA row is never stored
  const bool decoder = warp < active;
  const bool partial = (K & 127) != 0;
  const uint32_t pmax = (uint32_t)(K & 127) / 16u;  // threads that hold weights in a short last tile
  const uint32_t ring = ring_at + warp * RING + lane * 16u, to_codes = 512u - lane * 8u;
  const uint8_t *praw = a.w.raw + srow * K + p * 16u;
  const uint8_t *pcode = reinterpret_cast<const uint8_t *>(a.w.codes) + srow * ((int64_t)T * 64) + p * 8u;
  int pt = 0;  // first tile the load side has not asked for
  // the next tile into the slot at `at`, as one cp.async group (an empty group past the row's
  // end, so that "all but the newest D - 1 groups" always names the tile being decoded); in a
  // short last tile the threads past the row's end copy thread 0's bytes and ignore them
  auto load_tile = [&](uint32_t at) {
    if (pt < T) {
      const bool tail = partial && pt == T - 1 && p >= pmax;
      copy_tile<R, 0>(at, to_codes, tail ? praw - p * 16u : praw, pcode, true, 0.0f);
      praw += 128, pcode += 64, pt++;
    }
    cp_commit();
  };
  if (decoder) {
#pragma unroll
    for (int u = 0; u < D; u++) load_tile(ring + u * SLOT);
  }

  build_pair_lut(reinterpret_cast<uint32_t *>(gen + (lut_at - base)), a.w.table);  // syncs once inside
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem) : "r"(win.slot));

  bool ok = true;

  if (decoder) {
    OctSelf me;
    asm volatile("mov.u32 %0, 0;" : "=r"(me.ready)::"memory");  // after the barrier: orders the table reads
    me.lane = lane, me.lane_hi = lane & ~7u, me.to_codes = to_codes, me.lut = lut_at + lane * 4u;
    me.gmask = 0xFFu << (grp * 8u), me.ltg = me.gmask & lanemask_lt();
    me.esc = a.w.esc, me.esc_cap = a.w.n_esc + 1, me.esc_cols = a.w.esc_cols;
    const uint8_t *const flags = a.w.flags + srow * T;
    uint32_t epos = __ldg(a.w.row_esc + srow);
    EscWindow ew{};
    EscStream col[2]{};  // with column-ordered escapes: this thread's columns 2p and 2p + 1
    if constexpr (COLS) {
      const uint32_t starts = __ldg(reinterpret_cast<const uint32_t *>(a.w.col_esc + srow * 16) + p);
      stream_open(col[0], a.w.esc_cols, epos + (starts & 0xFFFFu));
      stream_open(col[1], a.w.esc_cols, epos + (starts >> 16));
    } else {
      ew.base = epos & ~3u;
      ew.word = window_load(me.esc, me.esc_cap, ew.base + p * 4u);
    }
    uint32_t nflag = p < 8u && (int)p < T ? (uint32_t)__ldg(flags + p) : 0u;  // this thread's flag byte of the next block of eight tiles
    uint32_t fm = 0;
    // the two 16-byte chunks of this thread in a stage: k 16p .. 16p+7 and 16p+8 .. 16p+15 of row r
    const uint32_t a_off0 = (p >> 2) * (MMA_BM * 128u) + swz(r, 2u * (p & 3u)), a_off1 = (p >> 2) * (MMA_BM * 128u) + swz(r, 2u * (p & 3u) + 1u);
    int s = 0;
    uint32_t ph = 1;  // parity of the `empty` phase that frees slot s (first pass: slots start free)
    // D tiles a round, so that tile ct + u sits in slot u (an immediate offset)
    for (int c0 = 0; c0 < T; c0 += D) {
#pragma unroll
      for (int u = 0; u < D; u++) {
        const int ct = c0 + u;
        if (ct >= T) break;
        const uint32_t at = ring + u * SLOT;
        if ((ct & 7) == 0) {  // a new block of eight tiles: fold the flag bytes, fetch the next block's
          const uint32_t v = __ballot_sync(BN_FULL, nflag != 0);
          fm = (v | (v >> 8) | (v >> 16) | (v >> 24)) & 0xFFu;
          const int nt = ct + 8 + (int)p;
          nflag = p < 8u && nt < T ? (uint32_t)__ldg(flags + nt) : 0u;
        }
        const uint32_t token = cp_wait<D - 1>();  // all but the newest D - 1 groups have landed: this tile's has
        uint32_t rr[R], cc[Geo::NC], w[2 * R];
        asm("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(rr[0]), "=r"(rr[1]), "=r"(rr[2]), "=r"(rr[3]) : "r"(at), "r"(token));
        asm("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(cc[0]), "=r"(cc[1]) : "r"(at + to_codes), "r"(token));
#pragma unroll
        for (int i = 0; i < R; i++) {
          const uint32_t c = (i & 1) ? cc[i >> 1] >> 16 : cc[i >> 1];
          w[2 * i] = (__byte_perm(rr[i], 0u, 0x1100) & 0x807F807Fu) | lut_read(me.lut + ((c << 7) & 0x7F80u), me.ready);
          w[2 * i + 1] = (__byte_perm(rr[i], 0u, 0x3322) & 0x807F807Fu) | lut_read(me.lut + ((c >> 1) & 0x7F80u), me.ready);
        }
        if ((fm >> (ct & 7)) & 1u) {
          if constexpr (COLS) {
            const uint32_t h0 = hits15(cc[0]), h1 = hits15(cc[1]);
            if (h0) stream_patch<0>(h0, col[0], a.w.esc_cols, w);
            if (h1) stream_patch<4>(h1, col[1], a.w.esc_cols, w);
          } else {
            oct_patch<R>(epos, ew, w, cc, me);
          }
        }
        if (partial && ct == T - 1 && p >= pmax) {  // past the row's end: zeros (the columns of X there are zeros too, but 0 x Inf must not happen)
#pragma unroll
          for (int i = 0; i < 2 * R; i++) w[i] = 0u;
        }
        if (ct >= S && ok) ok = mm_bar_wait(win.empty + 8 * s, ph);
        tc_fence_after();
        const uint32_t a_s = a_at + (uint32_t)s * MMA_A_STAGE;
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(a_s + a_off0), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(a_s + a_off1), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
        fence_async_smem();  // the tensor core reads shared memory through the async proxy
        __syncwarp();
        if (lane == 0) mm_bar_arrive(win.full + 8 * s);
        if (++s == S) s = 0, ph ^= 1u;
        load_tile(at);  // the slot just read takes the tile D further on
      }
    }
    cp_wait<0>();
  } else if (warp == MAXW) {
    ok = mma_issue_side(&x_map, win, T, S, BN, a.slice_tiles, tmem, lane, ok);
  }
  if (warp < 4) mma_store_side(a, win, tmem, warp, lane, row_base, rows, ok);
  tc_fence_before();
  __syncthreads();
  if (warp == MAXW) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(a.tmem_cols) : "memory");
}

typedef CUresult (*TensorMapEncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static TensorMapEncodeFn tensor_map_encoder() {
  static TensorMapEncodeFn fn = nullptr;
  if (!fn) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = (TensorMapEncodeFn)p;
  }
  return fn;
}

static int mma_sms() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

// Fused decode GEMM for up to 256 input rows (the MMA's largest N); -1 when the shape is outside its coverage.
int mma_rows(const bn_r4 *w, const uint16_t *x, int64_t x_stride, int64_t M, int64_t N, int64_t K, uint16_t *y, int64_t y_stride, int split, cudaStream_t s) {
  if (M < 1 || M > 256 || K % 8 || x_stride % 8 || N < 1 || ((uintptr_t)x & 15)) return -1;
  if (split < 1 || tiles(K) % split || ((M + 15) / 16 * 16) * split > 512) return -1;  // whole tiles per slice, all accumulators in tensor memory
  TensorMapEncodeFn encode = tensor_map_encoder();
  if (!encode) return fail(BN_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  MmaArgs a{};
  a.w = *w, a.y = y, a.N = N, a.K = K, a.y_stride = y_stride;
  a.T = (int)tiles(K), a.M = (int)M, a.BN = (int)((M + 15) / 16 * 16);
  a.split = split, a.slice_tiles = a.T / split;
  a.tmem_cols = 32;
  while ((int)a.tmem_cols < a.BN * split) a.tmem_cols *= 2;
  // X as a 2-D tensor [M rows, K columns] of BF16; a box is 64 columns (one 128-byte swizzled row
  // each) of BN rows; rows past M and columns past K read as zeros
  CUtensorMap x_map;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M}, strides[1] = {(cuuint64_t)x_stride * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)a.BN}, elem[2] = {1, 1};
  if (encode(&x_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t *>(x), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return fail(BN_ERR_CUDA, "cuTensorMapEncodeTiled failed for the input rows");
  const uint32_t fixed = 1024 + LUT_WORDS * 4 + 256;  // alignment slack, pair table, barriers
  const uint32_t per_stage = MMA_A_STAGE + (uint32_t)a.BN * MMA_BK * 2u;
  // eight threads per row where the rings fit beside at least two stages
  if (K % 16 == 0 && !(((uintptr_t)w->raw | (uintptr_t)w->codes) & 15)) {
    constexpr int ow = MMA_OCT_WARPS;
    int64_t rows = (N + mma_sms() - 1) / mma_sms();
    rows = (rows + 3) / 4 * 4;
    if (rows > ow * 4) rows = ow * 4;
    a.rows = (int)rows;
    const unsigned grid = (unsigned)((N + rows - 1) / rows);
    for (int slots = 4; slots >= 3; slots--) {
      const uint32_t rings = (uint32_t)ow * slots * 768u;
      if (fixed + rings + 2 * per_stage > MMA_SMEM_MAX) continue;
      int stages = (int)((MMA_SMEM_MAX - fixed - rings) / per_stage);
      a.stages = stages > 4 ? 4 : stages;
      const uint32_t smem = fixed + rings + (uint32_t)a.stages * per_stage;
      const bool cols = w->esc_cols && w->col_esc && !(((uintptr_t)w->esc_cols | (uintptr_t)w->col_esc) & 3);
      auto kern = slots == 4 ? (cols ? r4_mma_oct_kernel<ow, 4, true> : r4_mma_oct_kernel<ow, 4, false>) : (cols ? r4_mma_oct_kernel<ow, 3, true> : r4_mma_oct_kernel<ow, 3, false>);
      BN_CUDA(allow_smem(kern, smem));
      kern<<<grid, (ow + 1) * 32, smem, s>>>(x_map, a);
      return launched("r4_mma_oct_kernel");
    }
  }
  // an equal share of the rows for every SM, in whole warps' worth of rows
  constexpr int dw = MMA_DECODE_WARPS, rpw = MMA_RPW;
  int64_t rows = (N + mma_sms() - 1) / mma_sms();
  rows = (rows + rpw - 1) / rpw * rpw;
  if (rows > dw * rpw) rows = dw * rpw;
  a.rows = (int)rows;
  int stages = (int)((MMA_SMEM_MAX - fixed) / per_stage);
  if (stages > 4) stages = 4;
  if (stages < 2) return -1;
  a.stages = stages;
  const uint32_t smem = fixed + (uint32_t)stages * per_stage;
  const unsigned grid = (unsigned)((N + rows - 1) / rows);
  BN_CUDA(allow_smem(r4_mma_kernel<dw, rpw>, smem));
  r4_mma_kernel<dw, rpw><<<grid, (dw + 1) * 32, smem, s>>>(x_map, a);
  return launched("r4_mma_kernel");
}

int mma_status_reset() {
  const int zero = 0;
  BN_CUDA(cudaMemcpyToSymbol(g_mma_error, &zero, sizeof(int)));
  return BN_OK;
}

int mma_status(int *status) {
  BN_CUDA(cudaMemcpyFromSymbol(status, g_mma_error, sizeof(int)));
  return BN_OK;
}

}  // namespace bn

extern "C" int bn_r4_mma_split(const uint16_t *x, int64_t x_stride, const bn_r4 *w, int64_t M, int64_t N, int64_t K, uint16_t *y, int64_t y_stride, int split, void *stream) {
  if (!w || !w->raw || !w->codes || !w->flags || !w->esc || !w->table || !w->row_esc) return bn::fail(BN_ERR_ARG, "bn_r4_mma: null R4 array");
  if (!x || !y || N < 0 || K <= 0 || M < 1 || M > 256) return bn::fail(BN_ERR_ARG, "bn_r4_mma: bad size (1 <= M <= 256) or null pointer");
  if (K % 8 || x_stride % 8) return bn::fail(BN_ERR_ARG, "bn_r4_mma needs K % 8 == 0 and x rows 16-byte aligned");
  if (split < 1) return bn::fail(BN_ERR_ARG, "bn_r4_mma_split: split must be at least 1");
  if (N == 0) return BN_OK;
  const int e = bn::mma_rows(w, x, x_stride, M, N, K, y, y_stride, split, (cudaStream_t)stream);
  return e == -1 ? bn::fail(BN_ERR_ARG, "bn_r4_mma: shape does not fit shared or tensor memory, or the K tiles do not divide into the slices") : e;
}

extern "C" int bn_r4_mma(const uint16_t *x, int64_t x_stride, const bn_r4 *w, int64_t M, int64_t N, int64_t K, uint16_t *y, int64_t y_stride, void *stream) {
  return bn_r4_mma_split(x, x_stride, w, M, N, K, y, y_stride, 1, stream);
}
