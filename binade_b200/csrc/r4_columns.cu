// Column-ordered escapes of an R4 matrix: the acceleration arrays `esc_cols` and `col_esc` of
// bn_r4, built once at load time from the standard arrays.
//
// In the standard layout a row's escape bytes follow weight order, so the position of a
// thread's escape depends on how many escapes the other threads of the row hold in the same
// tile: the batch-1 kernels have to agree on it with ballots for every flagged tile. Here the
// row's run of escape bytes is permuted so that the escapes of column c (weights k with
// (k % 128) / 8 == c: the eight weights of one 32-bit code word of every tile) are contiguous,
// columns in order 0..15; col_esc[r][c] is the start of column c inside row r's run. A thread
// that owns a column then needs nothing from its neighbours.
//
// Sixteen threads per row, one per column, two passes over the row's flagged tiles (found from
// the flag bytes, 32 tiles at a time): count, then copy. Load-time work.
#include "common.cuh"

namespace bn {
namespace {

__device__ __forceinline__ uint32_t col_hits15(uint32_t c) {
  const uint32_t t = c & (c >> 1);
  return t & (t >> 2) & 0x11111111u;
}

// inclusive sum over the 16 lanes of this thread's half of the warp
__device__ __forceinline__ uint32_t half_scan(uint32_t v, uint32_t c, uint32_t mask) {
#pragma unroll
  for (int d = 1; d < 16; d <<= 1) {
    const uint32_t n = __shfl_up_sync(mask, v, d, 16);
    if (c >= (uint32_t)d) v += n;
  }
  return v;
}

__global__ void __launch_bounds__(256) r4_esc_columns_kernel(const bn_r4 w, int64_t N, int T, uint8_t *__restrict__ out, uint16_t *__restrict__ col_esc) {
  const int64_t r = (int64_t)blockIdx.x * (blockDim.x / 16) + threadIdx.x / 16;
  const uint32_t c = threadIdx.x & 15u, half = threadIdx.x & 16u, mask = 0xFFFFu << half;
  if (r >= N) return;  // whole half-warps leave together
  const uint32_t *codes = reinterpret_cast<const uint32_t *>(w.codes) + r * (int64_t)T * 16 + c;  // the code word of column c in tile 0
  const uint8_t *flags = w.flags + r * (int64_t)T;
  // bit u of the result: tile t0 + u is flagged (every lane of the row gets the same word; only
  // the flagged tiles, one in eight on typical weights, are visited below)
  auto flagged = [&](int t0) {
    const uint32_t lo = t0 + (int)c < T ? flags[t0 + c] : 0u, hi = t0 + 16 + (int)c < T ? flags[t0 + 16 + c] : 0u;
    const uint32_t a = __ballot_sync(mask, lo != 0) >> half, b = __ballot_sync(mask, hi != 0) >> half;
    return (a & 0xFFFFu) | (b << 16);
  };
  uint32_t cnt = 0;
  for (int t0 = 0; t0 < T; t0 += 32)
    for (uint32_t m = flagged(t0); m; m &= m - 1) cnt += __popc(col_hits15(__ldg(codes + (t0 + __ffs(m) - 1) * 16)));
  const uint32_t start = half_scan(cnt, c, mask) - cnt;
  col_esc[r * 16 + c] = (uint16_t)start;
  const uint32_t base = w.row_esc[r];
  uint32_t src_tile = base, dst = base + start;
  for (int t0 = 0; t0 < T; t0 += 32)
    for (uint32_t m = flagged(t0); m; m &= m - 1) {
      const uint32_t n = __popc(col_hits15(__ldg(codes + (t0 + __ffs(m) - 1) * 16)));
      const uint32_t upto = half_scan(n, c, mask);
      uint32_t src = src_tile + upto - n;
      for (uint32_t i = 0; i < n; i++) out[dst++] = w.esc[src++];
      src_tile += __shfl_sync(mask, upto, 15, 16);
    }
}

}  // namespace
}  // namespace bn

extern "C" int bn_r4_esc_columns(const bn_r4 *w, int64_t N, int64_t K, uint8_t *esc_cols, uint16_t *col_esc, void *stream) {
  if (!w || !w->codes || !w->flags || !w->esc || !w->row_esc || !esc_cols || !col_esc) return bn::fail(BN_ERR_ARG, "bn_r4_esc_columns: null pointer");
  if (N < 0 || K <= 0 || K % 16 || K > 65520) return bn::fail(BN_ERR_ARG, "bn_r4_esc_columns needs K % 16 == 0 and K <= 65520");
  if (reinterpret_cast<uintptr_t>(w->codes) & 3) return bn::fail(BN_ERR_ARG, "bn_r4_esc_columns: codes must be 4-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  BN_CUDA(cudaMemsetAsync(esc_cols + w->n_esc, 0, 8, s));
  if (N == 0) return BN_OK;
  const int per_block = 256 / 16;
  bn::r4_esc_columns_kernel<<<(unsigned)((N + per_block - 1) / per_block), 256, 0, s>>>(*w, N, (int)bn::tiles(K), esc_cols, col_esc);
  return bn::launched("r4_esc_columns_kernel");
}
