// Rice (format 2) encoder on the GPU: BF16 words already on the device -> the file arrays
// (raw, meta, bits, roff), bit for bit what the host encoder and the reference's
// binade/rice.py:57-125 write. The reference encodes on the CPU with numpy (about a million
// weights a second); this is three passes over the tensor at memory speed.
//
//   bn_bf16_split_hist   raw byte (sign << 7 | mantissa) of every word and the histogram of the
//                        exponent bytes; the host turns the histogram into the rank table
//                        (binade/format.py:34-42: 256 entries, nothing to gain on a GPU)
//   bn_rice_encode_plan  per tile the Rice parameter k (0..3) with the smallest cost
//                        k n + sum min(q + 1, qmax), q = rank >> k, qmax = max q <= 63, ties to the
//                        smaller k (binade/rice.py:57-73) -> meta = k | qmax << 2; per row the
//                        stream's length in 32-bit words; then the rows' first words (exclusive
//                        prefix sum) and the total
//   bn_rice_encode_write the streams: one warp per row, lane l owns weights 4l .. 4l+3 of a tile
//                        (the decoder's ownership), the low plane and every unary plane placed by
//                        a warp prefix sum of the lanes' bit counts; bits are OR-ed into a window of
//                        the row's stream in shared memory and whole words flushed to global
//                        memory with coalesced stores
#include "common.cuh"

namespace bn {
namespace {

constexpr int ENC_THREADS = 256;
constexpr int ENC_WINDOW = 640;  // words of a row's stream a warp holds: a tile is at most 265 words (128 x (3 + 63) bits + a partial word)

__global__ void __launch_bounds__(256) split_hist_kernel(const uint16_t *__restrict__ w, int64_t n, uint8_t *__restrict__ raw, uint32_t *__restrict__ hist) {
  __shared__ uint32_t h[256];
  h[threadIdx.x] = 0;
  __syncthreads();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const uint32_t v = w[i];
    raw[i] = (uint8_t)(((v >> 8) & 0x80u) | (v & 0x7Fu));
    atomicAdd(&h[(v >> 7) & 0xFFu], 1u);
  }
  __syncthreads();
  if (h[threadIdx.x]) atomicAdd(hist + threadIdx.x, h[threadIdx.x]);
}

// ranks of the lane's four weights of tile t (weights past the row's end: rank 0, not real)
__device__ __forceinline__ void lane_ranks(const uint16_t *__restrict__ row, const uint8_t *rank, int64_t K, int t, uint32_t lane, uint32_t (&r)[4], uint32_t &nv) {
  const int64_t col = (int64_t)t * BN_TILE + lane * 4;
  nv = (uint32_t)max((int64_t)0, min((int64_t)4, K - col));
#pragma unroll
  for (int i = 0; i < 4; i++) r[i] = (uint32_t)i < nv ? rank[(row[col + i] >> 7) & 0xFFu] : 0u;
}

// (k, qmax, bits) of a tile from the lanes' ranks; whole warp calls it
__device__ __forceinline__ void choose(const uint32_t (&r)[4], uint32_t nv, uint32_t n, uint32_t &k_best, uint32_t &qmax_best, uint32_t &bits_best) {
  bits_best = 0xFFFFFFFFu, k_best = 0, qmax_best = 0;
  const uint32_t rmax = __reduce_max_sync(BN_FULL, max(max(r[0], r[1]), max(r[2], r[3])));
#pragma unroll
  for (uint32_t k = 0; k < 4; k++) {
    const uint32_t qm = rmax >> k;
    uint32_t c = 0;
#pragma unroll
    for (int i = 0; i < 4; i++)
      if ((uint32_t)i < nv) c += min((r[i] >> k) + 1u, qm);
    c = __reduce_add_sync(BN_FULL, c) + k * n;
    if (qm <= 63u && c < bits_best) bits_best = c, k_best = k, qmax_best = qm;  // strict: ties keep the smaller k
  }
}

__global__ void __launch_bounds__(ENC_THREADS) plan_kernel(const uint16_t *__restrict__ w, const uint8_t *__restrict__ rank_table, int64_t R, int64_t K, int T, uint8_t *__restrict__ meta, uint32_t *__restrict__ row_words) {
  __shared__ uint8_t rank[256];
  rank[threadIdx.x] = rank_table[threadIdx.x];
  __syncthreads();
  const uint32_t lane = lane_id();
  const int warps = ENC_THREADS / 32;
  for (int64_t row = (int64_t)blockIdx.x * warps + (threadIdx.x >> 5); row < R; row += (int64_t)gridDim.x * warps) {
    const uint16_t *src = w + row * K;
    uint64_t bits = 0;
    for (int t = 0; t < T; t++) {
      uint32_t r[4], nv, k, qmax, c;
      lane_ranks(src, rank, K, t, lane, r, nv);
      choose(r, nv, (uint32_t)min((int64_t)BN_TILE, K - (int64_t)t * BN_TILE), k, qmax, c);
      if (lane == 0) meta[row * T + t] = (uint8_t)(k | (qmax << 2));
      bits += c;
    }
    if (lane == 0) row_words[row] = (uint32_t)min((bits + 31) >> 5, (uint64_t)0xFFFFFFFFu);
  }
}

// roff = exclusive prefix sum of row_words (one block, the rows in order); total[0] = number of
// words as uint64 (a total of 2^32 or more cannot be addressed by the format's uint32 offsets:
// the caller checks)
__global__ void __launch_bounds__(1024) offsets_kernel(const uint32_t *__restrict__ row_words, int64_t R, uint32_t *__restrict__ roff, unsigned long long *__restrict__ total) {
  __shared__ unsigned long long warp_sum[32];
  __shared__ unsigned long long carry;
  const uint32_t lane = lane_id(), warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int64_t base = 0; base < R; base += 1024) {
    const int64_t i = base + threadIdx.x;
    const unsigned long long v = i < R ? row_words[i] : 0ull;
    unsigned long long inc = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const unsigned long long n = __shfl_up_sync(BN_FULL, inc, d);
      if (lane >= (uint32_t)d) inc += n;
    }
    if (lane == 31) warp_sum[warp] = inc;
    __syncthreads();
    unsigned long long before = carry;
    for (uint32_t j = 0; j < warp; j++) before += warp_sum[j];
    if (i < R) roff[i] = (uint32_t)(before + inc - v);
    __syncthreads();
    if (threadIdx.x == 1023) carry = before + inc;
    __syncthreads();
  }
  if (threadIdx.x == 0) *total = carry;
}

// OR `n` <= 32 bits into the window at bit `pos` (counted from the window's first word)
__device__ __forceinline__ void put_bits(uint32_t *win, uint32_t pos, uint32_t v, uint32_t n) {
  if (!n) return;
  const uint32_t wi = pos >> 5, s = pos & 31u;
  atomicOr(win + wi, v << s);
  if (s + n > 32u) atomicOr(win + wi + 1, v >> (32u - s));
}

__global__ void __launch_bounds__(ENC_THREADS) write_kernel(const uint16_t *__restrict__ w, const uint8_t *__restrict__ rank_table, const uint8_t *__restrict__ meta, const uint32_t *__restrict__ roff, int64_t R, int64_t K, int T, uint32_t *__restrict__ bits, uint64_t nwords) {
  __shared__ uint8_t rank[256];
  __shared__ uint32_t window[ENC_THREADS / 32][ENC_WINDOW];
  rank[threadIdx.x] = rank_table[threadIdx.x];
  __syncthreads();
  const uint32_t lane = lane_id(), lt = lanemask_lt();
  const int warps = ENC_THREADS / 32;
  uint32_t *win = window[threadIdx.x >> 5];
  for (int64_t row = (int64_t)blockIdx.x * warps + (threadIdx.x >> 5); row < R; row += (int64_t)gridDim.x * warps) {
    const uint16_t *src = w + row * K;
    uint32_t *dst = bits + roff[row];
    const uint64_t room = roff[row] < nwords ? nwords - roff[row] : 0;  // never write past the array
    for (int i = lane; i < ENC_WINDOW; i += 32) win[i] = 0;
    __syncwarp();
    uint32_t cur = 0;   // bits of the row written so far
    uint32_t base = 0;  // the window's first word, as a word index of the row
    for (int t = 0; t < T; t++) {
      // whole words behind the cursor are final: flush them when the next tile might not fit
      if ((cur >> 5) - base + 266u > (uint32_t)ENC_WINDOW) {
        const uint32_t done = (cur >> 5) - base;
        for (uint32_t i = lane; i < done; i += 32)
          if ((uint64_t)base + i < room) dst[base + i] = win[i];
        __syncwarp();
        const uint32_t last = win[done];  // the partial word moves to the front
        __syncwarp();
        for (int i = lane; i < ENC_WINDOW; i += 32) win[i] = i == 0 ? last : 0u;
        __syncwarp();
        base += done;
      }
      uint32_t r[4], nv;
      lane_ranks(src, rank, K, t, lane, r, nv);
      const uint32_t m = meta[row * T + t], k = m & 3u, qmax = m >> 2, km = (1u << k) - 1u;
      const uint32_t n = (uint32_t)min((int64_t)BN_TILE, K - (int64_t)t * BN_TILE);
      const uint32_t at = cur - (base << 5);  // the tile's first bit inside the window
      // low plane: weight i's k bits at i k
      uint32_t lo = 0;
#pragma unroll
      for (int i = 0; i < 4; i++)
        if ((uint32_t)i < nv) lo |= (r[i] & km) << (i * k);
      put_bits(win, at + lane * 4u * k, lo, nv * k);
      uint32_t plane_at = at + n * k;
      // unary planes: one bit per weight still alive (q >= j), set iff q > j
      uint32_t q[4];
#pragma unroll
      for (int i = 0; i < 4; i++) q[i] = r[i] >> k;
      for (uint32_t j = 0; j < qmax; j++) {
        uint32_t v = 0, c = 0;
#pragma unroll
        for (int i = 0; i < 4; i++)
          if ((uint32_t)i < nv && q[i] >= j) v |= (q[i] > j ? 1u : 0u) << c, c++;
        const uint32_t b0 = __ballot_sync(BN_FULL, c & 1u), b1 = __ballot_sync(BN_FULL, c & 2u), b2 = __ballot_sync(BN_FULL, c & 4u);
        const uint32_t pre = __popc(b0 & lt) + 2 * __popc(b1 & lt) + 4 * __popc(b2 & lt);
        const uint32_t tot = __popc(b0) + 2 * __popc(b1) + 4 * __popc(b2);
        put_bits(win, plane_at + pre, v, c);
        plane_at += tot;
      }
      cur += plane_at - at;
      __syncwarp();
    }
    const uint32_t words = ((cur + 31u) >> 5) - base;
    for (uint32_t i = lane; i < words; i += 32)
      if ((uint64_t)base + i < room) dst[base + i] = win[i];
    __syncwarp();
  }
}

int enc_grid(int64_t R) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t blocks = (R + ENC_THREADS / 32 - 1) / (ENC_THREADS / 32), cap = (int64_t)sms * 8;
  return (int)max((int64_t)1, min(blocks, cap));
}

}  // namespace
}  // namespace bn

extern "C" int bn_bf16_split_hist(const uint16_t *w, int64_t n, uint8_t *raw, uint32_t *hist, void *stream) {
  if (!w || !raw || !hist || n < 0) return bn::fail(BN_ERR_ARG, "bn_bf16_split_hist: null pointer or negative size");
  cudaStream_t s = (cudaStream_t)stream;
  BN_CUDA(cudaMemsetAsync(hist, 0, 256 * sizeof(uint32_t), s));
  if (n == 0) return BN_OK;
  const int64_t want = (n + 255) / 256, blocks = want < 148 * 16 ? want : 148 * 16;
  bn::split_hist_kernel<<<(unsigned)blocks, 256, 0, s>>>(w, n, raw, hist);
  return bn::launched("split_hist_kernel");
}

extern "C" int bn_rice_encode_plan(const uint16_t *w, const uint8_t *rank, int64_t R, int64_t K, uint8_t *meta, uint32_t *row_words, uint32_t *roff, uint64_t *total, void *stream) {
  if (!w || !rank || !meta || !row_words || !roff || !total || R < 0 || K <= 0) return bn::fail(BN_ERR_ARG, "bn_rice_encode_plan: null pointer or bad size");
  cudaStream_t s = (cudaStream_t)stream;
  if (R == 0) {
    BN_CUDA(cudaMemsetAsync(total, 0, sizeof(uint64_t), s));
    return BN_OK;
  }
  bn::plan_kernel<<<bn::enc_grid(R), bn::ENC_THREADS, 0, s>>>(w, rank, R, K, (int)bn::tiles(K), meta, row_words);
  if (int e = bn::launched("plan_kernel")) return e;
  bn::offsets_kernel<<<1, 1024, 0, s>>>(row_words, R, roff, reinterpret_cast<unsigned long long *>(total));
  return bn::launched("offsets_kernel");
}

extern "C" int bn_rice_encode_write(const uint16_t *w, const uint8_t *rank, const uint8_t *meta, const uint32_t *roff, int64_t R, int64_t K, uint32_t *bits, uint64_t nwords, void *stream) {
  if (!w || !rank || !meta || !roff || (!bits && nwords) || R < 0 || K <= 0) return bn::fail(BN_ERR_ARG, "bn_rice_encode_write: null pointer or bad size");
  if (R == 0) return BN_OK;
  bn::write_kernel<<<bn::enc_grid(R), bn::ENC_THREADS, 0, (cudaStream_t)stream>>>(w, rank, meta, roff, R, K, (int)bn::tiles(K), bits, nwords);
  return bn::launched("write_kernel");
}
