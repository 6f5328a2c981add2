// Format-2 (Rice) stream decoders. One warp owns a row (tiles of a row are chained: a tile's
// length is only known once its planes are decoded); lane l owns weights 4l .. 4l+3 of every
// tile, so a lane's four ranks are exactly one R4 lane word (or one uint32 of 8-bit ranks).
//
// Stream of one tile (n weights, meta = k | qmax << 2):
//   low plane     n*k bits, bit b of weight i at i*k + b
//   unary planes  j = 0 .. qmax-1: one bit per weight still alive (q >= j), set iff q > j
// The bit offset of a lane inside a plane is the number of alive weights before it: a warp
// prefix sum over per-lane alive counts, done with three ballots. The expander of matrices with
// many rows maps several rows to a warp instead (rice_r4_wide_kernel, further down).
#include <atomic>

#include "common.cuh"

namespace bn {

enum RiceMode { RICE_RANKS = 0, RICE_UNPACK = 1, RICE_R4 = 2 };

struct RiceArgs {
  const uint8_t *meta;
  const uint32_t *bits;
  uint64_t nwords;
  const uint32_t *roff;
  const uint8_t *table;
  const uint8_t *raw;
  int64_t R, K;
  int T;
  // lookups (RICE_UNPACK only): output row i decodes stream row ids[i] of a table of `rows` rows
  const uint32_t *ids;
  int64_t rows;
  // format 1 (fixed-width codes, FMT == 1): `bits` is the index stream, `roff` the first word of
  // each row (bn_f1_offsets), f1_esc the file's escape bytes, f1_eoff the escapes before each row
  const uint8_t *f1_esc;
  uint64_t f1_nesc;
  const uint32_t *f1_eoff;
  // outputs
  uint32_t *ranks;   // RICE_RANKS: [R, T*32] four 8-bit ranks per word
  uint32_t *rend;    // RICE_RANKS / RICE_UNPACK: word after each row's last bit
  uint16_t *out;     // RICE_UNPACK: BF16 [R, K]
  uint16_t *codes;   // RICE_R4
  uint8_t *flags;    // RICE_R4
  uint32_t *row_cnt; // RICE_R4
  uint8_t *esc_tmp;  // RICE_R4 scratch
  uint64_t esc_cap;
  uint32_t *tmp_off;
  uint32_t *counters;
};

// n <= 32 bits of the stream starting at bit `pos`; words outside [0, nwords) read as zero.
__device__ __forceinline__ uint32_t read_bits(const uint32_t *__restrict__ bits, uint64_t nwords, uint64_t pos, uint32_t n) {
  const uint64_t w = pos >> 5;
  const uint32_t s = (uint32_t)pos & 31u;
  uint32_t lo = w < nwords ? __ldg(bits + w) : 0u;
  uint32_t hi = (s + n > 32u && w + 1 < nwords) ? __ldg(bits + w + 1) : 0u;
  uint32_t v = __funnelshift_r(lo, hi, s);
  return n >= 32u ? v : v & ((1u << n) - 1u);
}

// The same on a row: `row` points at the row's first word, `pos` counts bits from there, and
// `avail` words may be read (all 32-bit arithmetic: a row's stream is far below 2^32 bits).
__device__ __forceinline__ uint32_t row_bits(const uint32_t *__restrict__ row, uint32_t avail, uint32_t pos, uint32_t n) {
  const uint32_t w = pos >> 5, s = pos & 31u;
  uint32_t lo = w < avail ? __ldg(row + w) : 0u;
  uint32_t hi = (s + n > 32u && w + 1 < avail) ? __ldg(row + w + 1) : 0u;
  uint32_t v = __funnelshift_r(lo, hi, s);
  return n >= 32u ? v : v & ((1u << n) - 1u);
}

// Exclusive prefix over lanes and warp total of a per-lane count in 0..7: three ballots for the
// prefix, one warp reduction for the total. All 32 lanes must call.
__device__ __forceinline__ void warp_scan_count(uint32_t cnt, uint32_t lt, uint32_t &pre, uint32_t &tot) {
  const uint32_t b0 = __ballot_sync(BN_FULL, cnt & 1u), b1 = __ballot_sync(BN_FULL, cnt & 2u), b2 = __ballot_sync(BN_FULL, cnt & 4u);
  pre = __popc(b0 & lt) + 2 * __popc(b1 & lt) + 4 * __popc(b2 & lt);
  tot = __reduce_add_sync(BN_FULL, cnt);
}

constexpr int RICE_THREADS = 256;

// MODE: what is written (ranks, BF16 words, R4 arrays). FMT: how a tile is coded on file: 2 =
// Rice planes (binade/rice.py), 1 = fixed-width codes with escapes (binade/format.py:1-12: meta =
// b | escape << 4; a tile is exactly 4 b words, code i at bits i b ..; in escape mode the code
// 2^b - 1 stands for "next byte of the escape stream", an exponent, whose rank is looked up).
template <int MODE, int FMT = 2>
__global__ void __launch_bounds__(RICE_THREADS) rice_kernel(RiceArgs a) {
  __shared__ uint8_t tbl[256];
  __shared__ uint32_t inv[FMT == 1 ? 256 : 1];  // format 1: rank of an exponent (smallest rank listing it)
  if (FMT == 1) {
    inv[threadIdx.x] = 255u;
    __syncthreads();
    atomicMin(&inv[a.table[threadIdx.x]], threadIdx.x);
  }
  // deposit table: entry alive | bits << 4 spreads the low bits of `bits`, in order, over the
  // set positions of the 4-bit mask `alive` (a 4-bit pdep)
  __shared__ uint8_t deposit[256];
  {
    const uint32_t al = threadIdx.x & 15u;
    uint32_t b = threadIdx.x >> 4, out = 0;
    for (int i = 0; i < 4; i++)
      if ((al >> i) & 1u) out |= (b & 1u) << i, b >>= 1;
    deposit[threadIdx.x] = (uint8_t)out;
    if (MODE != RICE_RANKS || FMT == 1) tbl[threadIdx.x] = a.table[threadIdx.x];
    __syncthreads();
  }
  const uint32_t lane = lane_id(), lt = lanemask_lt();
  const int warps = RICE_THREADS / 32;
  const int T = a.T;
  const int64_t K = a.K;
  for (int64_t row = (int64_t)blockIdx.x * warps + (threadIdx.x >> 5); row < a.R; row += (int64_t)gridDim.x * warps) {
    const int64_t srow = (MODE == RICE_UNPACK && a.ids) ? (int64_t)a.ids[row] : row;  // row of the stream
    if (MODE == RICE_UNPACK && a.ids && srow >= a.rows) {  // an id outside the table: a row of zeros
      for (int64_t c = lane; c < K; c += 32) a.out[row * K + c] = 0;
      continue;
    }
    const int64_t srows = (MODE == RICE_UNPACK && a.ids) ? a.rows : a.R;
    const uint32_t w0 = a.roff[srow];
    const uint64_t w_end = srow + 1 < srows ? (uint64_t)a.roff[srow + 1] : a.nwords;
    // pull the row's stream toward the SM: one 128-byte line per lane, up to 4 KB
    {
      const uint64_t p = (uint64_t)w0 + lane * 32u;
      if (p < w_end && p < a.nwords) asm volatile("prefetch.global.L1 [%0];" ::"l"(a.bits + p));
    }
    const uint32_t *row_words = a.bits + w0;
    const uint32_t avail = (uint64_t)w0 < a.nwords ? (uint32_t)min(a.nwords - w0, (uint64_t)0xFFFFFFFFu) : 0u;
    uint32_t cur = 0;  // bits from the row's first word
    uint32_t f1_cur = FMT == 1 ? a.f1_eoff[srow] : 0u;  // format 1: cursor into the file's escape bytes
    uint32_t row_escapes = 0;
    uint64_t esc_base = 0;
    bool esc_room = false;
    if (MODE == RICE_R4) {
      // claim scratch for the most escapes the row's meta bytes allow: a tile can hold a rank
      // >= 15 only if its largest representable rank (qmax << k | low bits) reaches 15
      uint32_t bound = 0;
      for (int t = lane; t < T; t += 32) {
        const uint32_t m = a.meta[row * T + t], k = m & 3u, qmax = m >> 2;
        // format 1: a fixed tile reaches rank 15 from 4 bits on; an escaped weight may have any rank
        if (FMT == 1 ? ((m & 15u) >= 4u || (m & 16u)) : (((qmax << k) | ((1u << k) - 1u)) >= 15u)) bound += (uint32_t)min(BN_TILE, (int)K - t * BN_TILE);
      }
#pragma unroll
      for (int o = 16; o >= 1; o >>= 1) bound += __shfl_xor_sync(BN_FULL, bound, o);
      unsigned long long base = 0;
      if (lane == 0 && bound) base = atomicAdd(reinterpret_cast<unsigned long long *>(a.counters + 4), (unsigned long long)bound);
      base = __shfl_sync(BN_FULL, base, 0);
      esc_base = base;
      esc_room = base + bound <= a.esc_cap;
      if (lane == 0) a.tmp_off[row] = (uint32_t)base;
    }
    for (int t0 = 0; t0 < T; t0 += 32) {
      const uint32_t my_meta = t0 + (int)lane < T ? a.meta[srow * T + t0 + lane] : 0u;
      uint32_t my_flag = 0;
      const int tn = min(32, T - t0);
      for (int u = 0; u < tn; u++) {
        const int t = t0 + u;
        const uint32_t m = __shfl_sync(BN_FULL, my_meta, u);
        const int n = min(BN_TILE, (int)K - t * BN_TILE);
        const uint32_t nv = (uint32_t)max(0, min(4, n - (int)lane * 4));
        uint32_t r4 = 0;  // ranks of the lane's four weights, one per byte
        if (FMT == 1) {
          const uint32_t b = m & 15u, cm = (1u << b) - 1u;
          const uint32_t v = b ? row_bits(row_words, avail, cur + lane * 4u * b, 4u * b) : 0u;  // padding weights are coded too (as 0)
          cur += (uint32_t)BN_TILE * b;
          uint32_t c[4], hit = 0;
#pragma unroll
          for (int i = 0; i < 4; i++) {
            c[i] = (v >> (i * b)) & cm;
            if ((m & 16u) && c[i] == cm) hit |= 1u << i;
          }
          if (__any_sync(BN_FULL, hit != 0)) {
            uint32_t pre, tot;
            warp_scan_count(__popc(hit), lt, pre, tot);
            uint64_t q = (uint64_t)f1_cur + pre;
#pragma unroll
            for (int i = 0; i < 4; i++)
              if ((hit >> i) & 1u) {
                c[i] = q < a.f1_nesc ? inv[a.f1_esc[q]] : 0u;  // a short escape stream cannot be read past
                q++;
              }
            f1_cur += tot;
          }
          r4 = (c[0] & 0xFFu) | ((c[1] & 0xFFu) << 8) | ((c[2] & 0xFFu) << 16) | ((c[3] & 0xFFu) << 24);
        } else {
        const uint32_t k = m & 3u, qmax = m >> 2;
        uint32_t lo = 0;
        if (nv * k) lo = row_bits(row_words, avail, cur + lane * 4u * k, nv * k);
        cur += (uint32_t)n * k;
        uint32_t q4 = 0;  // one byte per weight
        uint32_t alive = (1u << nv) - 1u;
        for (uint32_t j = 0; j < qmax; j++) {
          const uint32_t c = __popc(alive);
          uint32_t pre, tot;
          warp_scan_count(c, lt, pre, tot);
          if (tot == 0) break;  // only a corrupt stream: the remaining planes are empty
          if (tot == 1) {
            // one weight left: its remaining planes are a run of ones closed by a zero (or by
            // reaching qmax); count it in one go instead of one warp scan per plane
            const uint32_t rem = qmax - j;
            uint32_t used = 0;
            if (c) {
              uint32_t ones = 0;
              for (uint32_t done = 0; done < rem; done += 32) {
                const uint32_t take = min(32u, rem - done);
                const uint32_t b = row_bits(row_words, avail, cur + done, take);
                const uint32_t run = __ffs(~b) - 1;  // 32 when b is all ones (ffs(0) = 0 wraps)
                if (run < take) { ones += run; break; }
                ones += take;
              }
              used = min(ones + 1, rem);
              q4 += ones << (8 * (__ffs(alive) - 1));
            }
            const uint32_t owner = __ffs(__ballot_sync(BN_FULL, c != 0)) - 1;
            cur += __shfl_sync(BN_FULL, used, owner);
            break;
          }
          const uint32_t b = c ? row_bits(row_words, avail, cur + pre, c) : 0u;
          alive = deposit[alive | (b << 4)];             // the plane's bits at the alive positions
          q4 += (alive * 0x00204081u) & 0x01010101u;     // bit i -> byte i: one more for the survivors
          cur += tot;
        }
        // ranks of the lane's four weights, one per byte: q << k | low bits
        const uint32_t km = (1u << k) - 1u;
#pragma unroll
        for (int i = 0; i < 4; i++) {
          const uint32_t r = ((((q4 >> (8 * i)) & 0xFFu) << k) | ((lo >> (i * k)) & km)) & 0xFFu;
          r4 |= r << (8 * i);
        }
        }
        if (MODE == RICE_RANKS) {
          a.ranks[(row * T + t) * 32 + lane] = r4;
        } else if (MODE == RICE_UNPACK) {
          const int64_t col = (int64_t)t * BN_TILE + lane * 4;
          if (nv == 4 && (K & 3) == 0) {  // aligned: one 4-byte load, one 8-byte store
            const uint32_t rw = ldg_stream_u32(a.raw + srow * K + col);
            uint32_t o[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
              const uint32_t b = (rw >> (8 * i)) & 0xFFu, e = tbl[(r4 >> (8 * i)) & 0xFFu];
              o[i] = ((b & 0x80u) << 8) | (e << 7) | (b & 0x7Fu);
            }
            *reinterpret_cast<uint2 *>(a.out + row * K + col) = make_uint2(o[0] | (o[1] << 16), o[2] | (o[3] << 16));
          } else {
            for (uint32_t i = 0; i < nv; i++) {
              const uint32_t b = a.raw[srow * K + col + i], e = tbl[(r4 >> (8 * i)) & 0xFFu];
              a.out[row * K + col + i] = (uint16_t)(((b & 0x80u) << 8) | (e << 7) | (b & 0x7Fu));
            }
          }
        } else {
          uint32_t c16 = 0, hit = 0;
#pragma unroll
          for (int i = 0; i < 4; i++) {
            const uint32_t r = (r4 >> (8 * i)) & 0xFFu;
            c16 |= min(r, 15u) << (4 * i);
            hit |= (r >= 15u ? 1u : 0u) << i;
          }
          a.codes[(row * T + t) * 32 + lane] = (uint16_t)c16;
          const uint32_t any = __ballot_sync(BN_FULL, hit != 0);
          if (any) {
            uint32_t pre, tot;
            warp_scan_small(__popc(hit), lt, pre, tot);
            if (esc_room) {
              uint64_t p = esc_base + row_escapes + pre;
#pragma unroll
              for (int i = 0; i < 4; i++)
                if ((hit >> i) & 1u) a.esc_tmp[p++] = tbl[(r4 >> (8 * i)) & 0xFFu];
            }
            row_escapes += tot;
            if ((int)lane == u) my_flag = 1;
          }
        }
      }
      if (MODE == RICE_R4 && t0 + (int)lane < T) a.flags[row * T + t0 + lane] = (uint8_t)my_flag;
    }
    if (lane == 0) {
      const uint32_t rend = w0 + ((cur + 31u) >> 5);
      if (MODE == RICE_R4) {
        a.row_cnt[row] = row_escapes;
        if (row_escapes) atomicAdd(a.counters + 2, row_escapes);
        if ((uint64_t)rend != w_end) atomicMax(a.counters + 1, (uint32_t)(a.R - row));
      } else if (a.rend) {
        a.rend[row] = rend;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Rice stream -> R4 arrays with several rows per warp (the expander's kernel for matrices with
// enough rows). A row's tiles are a chain and a plane of a tile is a chain too, so the decode is
// bound by the instructions it issues per plane step, not by bytes; the one-row-per-warp kernel
// above spends a whole warp instruction stream on every plane step of one row, and in the late
// planes only a handful of its 128 weights are still alive. Here LPR lanes own a row (8 lanes x
// 16 weights, or 16 lanes x 8), so one plane step of the warp serves 4 (or 2) rows: the scan over
// alive counts is a shuffle scan inside the LPR lanes, a lane deposits its up to 16 plane bits
// through the 4-bit deposit table nibble by nibble, and ranks, codes and escape tests are done
// four weights at a time on bytes packed in a register. The warp's rows walk their tiles in step
// (same tile index, their own bit cursors); a plane loop runs to the largest qmax of the warp's
// rows and ends early once no lane holds a live weight.
// Rows past R repeat row R-1 and write nothing. Blocks are two warps: with larger blocks the SMs
// of a launch end up with 24 or 32 warps each (three or four blocks) and the launch waits for the
// fuller ones.
// ---------------------------------------------------------------------------------------------
constexpr int RICE_WIDE_THREADS = 64;

template <int LPR>
__global__ void __launch_bounds__(RICE_WIDE_THREADS) rice_r4_wide_kernel(RiceArgs a) {
  constexpr int RPW = 32 / LPR;    // rows per warp
  constexpr int WPL = 128 / LPR;   // weights per lane and tile
  constexpr int NIB = WPL / 4;     // registers of four byte-packed weights
  __shared__ uint8_t tbl[256];
  __shared__ uint8_t deposit[256];  // alive | bits << 4 -> the low bits of `bits`, in order, on the set positions of `alive`
  for (uint32_t e = threadIdx.x; e < 256; e += RICE_WIDE_THREADS) {
    const uint32_t al = e & 15u;
    uint32_t b = e >> 4, out = 0;
    for (int i = 0; i < 4; i++)
      if ((al >> i) & 1u) out |= (b & 1u) << i, b >>= 1;
    deposit[e] = (uint8_t)out;
    tbl[e] = a.table[e];
  }
  __syncthreads();
  const uint32_t lane = lane_id(), p = lane & (LPR - 1), first = lane & ~(uint32_t)(LPR - 1);
  const int warps = RICE_WIDE_THREADS / 32;
  const int T = a.T;
  const int64_t K = a.K;
  // inclusive sum over the LPR lanes of a row
  auto row_scan = [&](uint32_t v) {
#pragma unroll
    for (int d = 1; d < LPR; d <<= 1) {
      const uint32_t n = __shfl_up_sync(BN_FULL, v, d, LPR);
      if (p >= (uint32_t)d) v += n;
    }
    return v;
  };
  for (int64_t row0 = ((int64_t)blockIdx.x * warps + (threadIdx.x >> 5)) * RPW; row0 < a.R; row0 += (int64_t)gridDim.x * warps * RPW) {
    const bool valid = row0 + lane / LPR < a.R;
    const int64_t row = valid ? row0 + lane / LPR : a.R - 1;
    const uint32_t w0 = a.roff[row];
    const uint64_t w_end = row + 1 < a.R ? (uint64_t)a.roff[row + 1] : a.nwords;
    const uint32_t *row_words = a.bits + w0;
    const uint32_t avail = (uint64_t)w0 < a.nwords ? (uint32_t)min(a.nwords - w0, (uint64_t)0xFFFFFFFFu) : 0u;
    // pull the row's stream toward the SM: one 128-byte line per lane and round, up to 4 KB a row
    for (uint32_t i = 0; i < 4096u / (LPR * 128u); i++) {
      const uint64_t at = (uint64_t)w0 + (i * LPR + p) * 32u;
      if (at < w_end && at < a.nwords) asm volatile("prefetch.global.L1 [%0];" ::"l"(a.bits + at));
    }
    // scratch for the most escapes the row's meta bytes allow (a tile can hold a rank >= 15 only
    // if its largest representable rank reaches 15)
    uint32_t bound = 0;
    for (int t = (int)p; t < T; t += LPR) {
      const uint32_t m = a.meta[row * T + t], k = m & 3u, qmax = m >> 2;
      if (((qmax << k) | ((1u << k) - 1u)) >= 15u) bound += (uint32_t)min(BN_TILE, (int)K - t * BN_TILE);
    }
#pragma unroll
    for (int o = LPR / 2; o >= 1; o >>= 1) bound += __shfl_xor_sync(BN_FULL, bound, o);
    unsigned long long base = 0;
    if (p == 0 && valid && bound) base = atomicAdd(reinterpret_cast<unsigned long long *>(a.counters + 4), (unsigned long long)bound);
    base = __shfl_sync(BN_FULL, base, first);
    const uint64_t esc_base = base;
    const bool esc_room = base + bound <= a.esc_cap;
    if (p == 0 && valid) a.tmp_off[row] = (uint32_t)base;

    uint32_t cur = 0, row_escapes = 0;
    uint32_t m_next = a.meta[row * T];
    for (int t = 0; t < T; t++) {
      const uint32_t m = m_next;
      if (t + 1 < T) m_next = a.meta[row * T + t + 1];
      const uint32_t k = m & 3u, qmax = m >> 2, km = (1u << k) - 1u;
      const int n = min(BN_TILE, (int)K - t * BN_TILE);
      const uint32_t nv = (uint32_t)max(0, min(WPL, n - (int)p * WPL));
      // low bits of the lane's weights: nv * k <= 48 bits
      const uint32_t nb = nv * k, lo_at = cur + p * WPL * k;
      uint32_t lo0 = nb ? row_bits(row_words, avail, lo_at, min(nb, 32u)) : 0u;
      uint32_t lo1 = nb > 32u ? row_bits(row_words, avail, lo_at + 32u, nb - 32u) : 0u;
      cur += (uint32_t)n * k;
      // unary planes
      uint32_t q[NIB];
#pragma unroll
      for (int i = 0; i < NIB; i++) q[i] = 0u;
      uint32_t alive = (1u << nv) - 1u;
      uint32_t planes = qmax;  // the warp runs to the largest qmax of its rows
#pragma unroll
      for (int o = 16; o >= LPR; o >>= 1) planes = max(planes, __shfl_xor_sync(BN_FULL, planes, o));
      for (uint32_t j = 0; j < planes; j++) {
        if (j >= qmax) alive = 0u;  // a weight alive after the last plane has q = qmax: nothing more to read
        const uint32_t c = __popc(alive);
        if (!__any_sync(BN_FULL, c != 0)) break;
        const uint32_t upto = row_scan(c), tot = __shfl_sync(BN_FULL, upto, first + LPR - 1);
        if (!__any_sync(BN_FULL, tot > 1u)) {
          // every row has at most one weight left: its remaining planes are a run of ones closed
          // by a zero (or by reaching qmax); count it in one go
          uint32_t used = 0;
          if (c) {
            const uint32_t rem = qmax - j;
            uint32_t ones = 0;
            for (uint32_t done = 0; done < rem; done += 32) {
              const uint32_t take = min(32u, rem - done);
              const uint32_t b = row_bits(row_words, avail, cur + done, take);
              const uint32_t run = __ffs(~b) - 1;  // 32 when b is all ones (ffs(0) = 0 wraps)
              if (run < take) { ones += run; break; }
              ones += take;
            }
            used = min(ones + 1, rem);
            const uint32_t i = __ffs(alive) - 1;
#pragma unroll
            for (int r = 0; r < NIB; r++)
              if ((i >> 2) == (uint32_t)r) q[r] += ones << (8 * (i & 3u));
          }
          const uint32_t holders = __ballot_sync(BN_FULL, c != 0) & (((LPR == 32 ? 0u : (1u << LPR)) - 1u) << first);
          const uint32_t owner = holders ? __ffs(holders) - 1 : lane;
          cur += __shfl_sync(BN_FULL, used, owner);
          break;
        }
        uint32_t b = c ? row_bits(row_words, avail, cur + upto - c, c) : 0u;
        uint32_t next = 0;
#pragma unroll
        for (int r = 0; r < NIB; r++) {
          const uint32_t al = (alive >> (4 * r)) & 15u;
          const uint32_t d = deposit[al | ((b & 15u) << 4)];  // the plane's bits at the alive positions
          b >>= __popc(al);
          next |= d << (4 * r);
          q[r] += (d * 0x00204081u) & 0x01010101u;  // bit i -> byte i: one more for the survivors
        }
        alive = next;
        cur += tot;
      }
      // ranks, codes and escape tests, four weights (bytes of a register) at a time
      uint32_t code_words[NIB / 2 > 0 ? NIB / 2 : 1], rank4[NIB], hit = 0;
#pragma unroll
      for (int r = 0; r < NIB; r++) {
        // the four weights' low bits, k each, spread to one byte each
        const uint32_t x = lo0 & ((1u << (4 * k)) - 1u);
        lo0 = __funnelshift_r(lo0, lo1, 4 * k), lo1 >>= 4 * k;
        const uint32_t pair0 = x & ((1u << (2 * k)) - 1u), pair1 = x >> (2 * k);
        const uint32_t both = km | (km << 8);
        const uint32_t low4 = ((pair0 | (pair0 << (8 - k))) & both) | (((pair1 | (pair1 << (8 - k))) & both) << 16);
        const uint32_t r4 = (((q[r] & ((0xFFu >> k) * 0x01010101u)) << k) | low4);
        rank4[r] = r4;
        // bit 7 of a byte of t: its rank is >= 15
        const uint32_t tt = (((r4 & 0x7F7F7F7Fu) + 0x71717171u) | r4) & 0x80808080u;
        const uint32_t full = (tt >> 7) * 15u;             // 0x0F in the bytes that escape
        uint32_t c4 = (r4 | full) & 0x0F0F0F0Fu;           // min(rank, 15) per byte
        c4 = (c4 | (c4 >> 4)) & 0x00FF00FFu;
        c4 = (c4 | (c4 >> 8)) & 0xFFFFu;                   // four nibbles
        if (r & 1) code_words[r >> 1] |= c4 << 16;
        else code_words[r >> 1] = c4;
        hit |= (((tt >> 7) * 0x00204081u >> 21) & 15u) << (4 * r);  // bytes' flags gathered into four bits
      }
      if (valid) {
        uint16_t *dst = a.codes + ((row * T + t) * 32 + p * (WPL / 4));
        if (NIB == 4) *reinterpret_cast<uint2 *>(dst) = make_uint2(code_words[0], code_words[NIB / 2 > 1 ? 1 : 0]);
        else *reinterpret_cast<uint32_t *>(dst) = code_words[0];
      }
      uint32_t flag = 0;
      if (__any_sync(BN_FULL, hit != 0)) {
        const uint32_t hc = __popc(hit), upto = row_scan(hc), tot = __shfl_sync(BN_FULL, upto, first + LPR - 1);
        if (valid && esc_room && hit) {
          uint64_t at = esc_base + row_escapes + upto - hc;
#pragma unroll
          for (int r = 0; r < NIB; r++)
#pragma unroll
            for (int i = 0; i < 4; i++)
              if ((hit >> (4 * r + i)) & 1u) a.esc_tmp[at++] = tbl[(rank4[r] >> (8 * i)) & 0xFFu];
        }
        row_escapes += tot;
        flag = tot != 0;
      }
      if (p == 0 && valid) a.flags[row * T + t] = (uint8_t)flag;
    }
    if (p == 0 && valid) {
      const uint32_t rend = w0 + ((cur + 31u) >> 5);
      a.row_cnt[row] = row_escapes;
      if (row_escapes) atomicAdd(a.counters + 2, row_escapes);
      if ((uint64_t)rend != w_end) atomicMax(a.counters + 1, (uint32_t)(a.R - row));
    }
  }
}

// row_esc = exclusive prefix sum of row_cnt, by one block (load-time, R up to a few 10^5).
__global__ void __launch_bounds__(1024) scan_rows_kernel(const uint32_t *row_cnt, int64_t R, uint32_t *row_esc) {
  __shared__ uint32_t part[1024];
  const int tid = threadIdx.x;
  const int64_t per = (R + 1023) / 1024, lo = min(R, per * tid), hi = min(R, lo + per);
  uint32_t s = 0;
  for (int64_t i = lo; i < hi; i++) s += row_cnt[i];
  part[tid] = s;
  __syncthreads();
  for (int o = 1; o < 1024; o <<= 1) {
    const uint32_t v = tid >= o ? part[tid - o] : 0u;
    __syncthreads();
    part[tid] += v;
    __syncthreads();
  }
  uint32_t run = part[tid] - s;
  for (int64_t i = lo; i < hi; i++) {
    const uint32_t c = row_cnt[i];  // read before the write: row_esc may alias row_cnt
    row_esc[i] = run;
    run += c;
  }
}

// esc[row_esc[r] + i] = esc_tmp[tmp_off[r] + i], i < (escapes of row r); one warp per row.
__global__ void __launch_bounds__(256) compact_esc_kernel(const uint32_t *__restrict__ row_esc, const uint8_t *__restrict__ esc_tmp, const uint32_t *__restrict__ tmp_off, int64_t R, uint8_t *__restrict__ esc, uint64_t esc_bytes) {
  const uint32_t lane = lane_id();
  for (int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); row < R; row += (int64_t)gridDim.x * 8) {
    const uint64_t b = row_esc[row], e = row + 1 < R ? (uint64_t)row_esc[row + 1] : esc_bytes - 1;
    const uint8_t *src = esc_tmp + tmp_off[row];
    for (uint64_t i = lane; b + i < e; i += 32) esc[b + i] = src[i];
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) esc[esc_bytes - 1] = 0;
}

// ---------------------------------------------------------------------------------------------
// Format 1 carries no row offsets: a tile of width b is 4 b words, escapes are one stream for the
// whole tensor. Two small passes rebuild, per row, the first index word and the escapes before it.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) f1_row_words_kernel(const uint8_t *__restrict__ meta, int64_t R, int T, uint32_t *__restrict__ words) {
  const uint32_t lane = lane_id();
  for (int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); row < R; row += (int64_t)gridDim.x * 8) {
    uint32_t n = 0;
    for (int t = lane; t < T; t += 32) n += 4u * (meta[row * T + t] & 15u);
    n = __reduce_add_sync(BN_FULL, n);
    if (lane == 0) words[row] = n;
  }
}

__global__ void __launch_bounds__(256) f1_row_escapes_kernel(const uint8_t *__restrict__ meta, const uint32_t *__restrict__ idx, uint64_t nwords, const uint32_t *__restrict__ woff, int64_t R, int T, uint32_t *__restrict__ count) {
  const uint32_t lane = lane_id();
  for (int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); row < R; row += (int64_t)gridDim.x * 8) {
    const uint32_t w0 = woff[row];
    const uint32_t avail = (uint64_t)w0 < nwords ? (uint32_t)min(nwords - w0, (uint64_t)0xFFFFFFFFu) : 0u;
    uint32_t cur = 0, n = 0;
    for (int t = 0; t < T; t++) {
      const uint32_t m = meta[row * T + t], b = m & 15u, cm = (1u << b) - 1u;
      if ((m & 16u) && b) {
        const uint32_t v = row_bits(idx + w0, avail, cur + lane * 4u * b, 4u * b);
#pragma unroll
        for (int i = 0; i < 4; i++) n += ((v >> (i * b)) & cm) == cm;
      }
      cur += (uint32_t)BN_TILE * b;
    }
    n = __reduce_add_sync(BN_FULL, n);
    if (lane == 0) count[row] = n;
  }
}

// totals[0] = index words, totals[1] = escapes the meta bytes and the index stream imply
__global__ void f1_totals_kernel(const uint32_t *woff, const uint32_t *words, const uint32_t *eoff, const uint32_t *count, int64_t R, uint32_t *totals) {
  totals[0] = woff[R - 1] + words[R - 1];
  totals[1] = eoff[R - 1] + count[R - 1];
}

static int rice_grid(int64_t R) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int64_t blocks = (R + RICE_THREADS / 32 - 1) / (RICE_THREADS / 32);
  const int64_t cap = (int64_t)sms * 8;
  return (int)(blocks < cap ? blocks : cap);
}

// The expander's kernel for R rows: four rows a warp when the matrix has rows for that on every
// SM, two from half of that, else one row a warp (the general kernel): fewer instructions per
// row against fewer warps to hide a plane step's latency.
static int launch_rice_r4(const RiceArgs &a, cudaStream_t s) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // measured on 3840-wide rows (ms, one / two / four rows a warp): 15360 rows 0.31 / 0.24 / 0.22,
  // 4096 rows 0.116 / 0.107 / 0.122, 2048 rows 0.077 / 0.095 / 0.116; 3840 rows of 15360: 0.39 / 0.35 / 0.40
  const int lpr = a.R >= (int64_t)sms * 48 ? 8 : a.R >= (int64_t)sms * 24 ? 16 : 32;
  if (lpr == 8 || lpr == 16) {
    const int64_t warps = (a.R * lpr + 31) / 32, per_block = RICE_WIDE_THREADS / 32;
    const int64_t blocks = min((warps + per_block - 1) / per_block, (int64_t)sms * 32);
    if (lpr == 8) rice_r4_wide_kernel<8><<<(unsigned)blocks, RICE_WIDE_THREADS, 0, s>>>(a);
    else rice_r4_wide_kernel<16><<<(unsigned)blocks, RICE_WIDE_THREADS, 0, s>>>(a);
    return launched("rice_r4_wide_kernel");
  }
  rice_kernel<RICE_R4><<<rice_grid(a.R), RICE_THREADS, 0, s>>>(a);
  return launched("rice_kernel<r4>");
}

static int check_stream(const uint8_t *meta, const uint32_t *bits, const uint32_t *roff, int64_t R, int64_t K) {
  if (!meta || !bits || !roff) return fail(BN_ERR_ARG, "null Rice stream array");
  if (R < 0 || K <= 0) return fail(BN_ERR_ARG, "bad matrix size");
  return BN_OK;
}

}  // namespace bn

using namespace bn;

extern "C" int bn_rice_ranks(const uint8_t *meta, const uint32_t *bits, uint64_t nwords, const uint32_t *roff, int64_t R, int64_t K, uint8_t *ranks, uint32_t *rend, void *stream) {
  if (int e = check_stream(meta, bits, roff, R, K)) return e;
  if (!ranks || !rend) return fail(BN_ERR_ARG, "bn_rice_ranks: null output");
  if (R == 0) return BN_OK;
  RiceArgs a{};
  a.meta = meta, a.bits = bits, a.nwords = nwords, a.roff = roff, a.R = R, a.K = K, a.T = (int)tiles(K);
  a.ranks = reinterpret_cast<uint32_t *>(ranks), a.rend = rend;
  rice_kernel<RICE_RANKS><<<rice_grid(R), RICE_THREADS, 0, (cudaStream_t)stream>>>(a);
  return launched("rice_kernel<ranks>");
}

extern "C" int bn_rice_unpack(const uint8_t *meta, const uint32_t *bits, uint64_t nwords, const uint32_t *roff, const uint8_t *table, const uint8_t *raw, int64_t R, int64_t K, uint16_t *out, uint32_t *rend, void *stream) {
  if (int e = check_stream(meta, bits, roff, R, K)) return e;
  if (!table || !raw || !out || !rend) return fail(BN_ERR_ARG, "bn_rice_unpack: null pointer");
  if (R == 0) return BN_OK;
  RiceArgs a{};
  a.meta = meta, a.bits = bits, a.nwords = nwords, a.roff = roff, a.table = table, a.raw = raw, a.R = R, a.K = K, a.T = (int)tiles(K);
  a.out = out, a.rend = rend;
  rice_kernel<RICE_UNPACK><<<rice_grid(R), RICE_THREADS, 0, (cudaStream_t)stream>>>(a);
  return launched("rice_kernel<unpack>");
}

extern "C" int bn_rice_lookup(const uint8_t *meta, const uint32_t *bits, uint64_t nwords, const uint32_t *roff, const uint8_t *table, const uint8_t *raw, int64_t rows, int64_t K, const uint32_t *ids, int64_t n, uint16_t *out, void *stream) {
  if (int e = check_stream(meta, bits, roff, rows, K)) return e;
  if (!table || !raw || !ids || !out || n < 0) return fail(BN_ERR_ARG, "bn_rice_lookup: null pointer or negative count");
  if (n == 0) return BN_OK;
  RiceArgs a{};
  a.meta = meta, a.bits = bits, a.nwords = nwords, a.roff = roff, a.table = table, a.raw = raw, a.R = n, a.K = K, a.T = (int)tiles(K);
  a.ids = ids, a.rows = rows, a.out = out, a.rend = nullptr;
  rice_kernel<RICE_UNPACK><<<rice_grid(n), RICE_THREADS, 0, (cudaStream_t)stream>>>(a);
  return launched("rice_kernel<unpack>");
}

extern "C" int bn_rice_to_r4(const uint8_t *meta, const uint32_t *bits, uint64_t nwords, const uint32_t *roff, const uint8_t *table, int64_t R, int64_t K, uint16_t *codes, uint8_t *flags, uint32_t *row_cnt, uint8_t *esc_tmp, uint64_t esc_cap, uint32_t *tmp_off, uint32_t *counters, void *stream) {
  if (int e = check_stream(meta, bits, roff, R, K)) return e;
  if (!table || !codes || !flags || !row_cnt || !tmp_off || !counters || (!esc_tmp && esc_cap)) return fail(BN_ERR_ARG, "bn_rice_to_r4: null pointer");
  if (K % 4) return fail(BN_ERR_ARG, "R4 needs K % 4 == 0");
  BN_CUDA(cudaMemsetAsync(counters, 0, 8 * sizeof(uint32_t), (cudaStream_t)stream));
  if (R == 0) return BN_OK;
  RiceArgs a{};
  a.meta = meta, a.bits = bits, a.nwords = nwords, a.roff = roff, a.table = table, a.R = R, a.K = K, a.T = (int)tiles(K);
  a.codes = codes, a.flags = flags, a.row_cnt = row_cnt, a.esc_tmp = esc_tmp, a.esc_cap = esc_cap, a.tmp_off = tmp_off, a.counters = counters;
  return launch_rice_r4(a, (cudaStream_t)stream);
}

extern "C" int bn_r4_finish(const uint32_t *row_cnt, const uint8_t *esc_tmp, const uint32_t *tmp_off, int64_t R, uint32_t *row_esc, uint8_t *esc, uint64_t esc_bytes, void *stream) {
  if (!row_cnt || !tmp_off || !row_esc || !esc || esc_bytes < 1 || R < 0) return fail(BN_ERR_ARG, "bn_r4_finish: null pointer or empty esc");
  if (!esc_tmp && esc_bytes > 1) return fail(BN_ERR_ARG, "bn_r4_finish: escapes without scratch");
  cudaStream_t s = (cudaStream_t)stream;
  if (R > 0) {
    scan_rows_kernel<<<1, 1024, 0, s>>>(row_cnt, R, row_esc);
    if (int e = launched("scan_rows_kernel")) return e;
  }
  int64_t blocks = (R + 7) / 8;
  if (blocks > 2048) blocks = 2048;
  if (blocks < 1) blocks = 1;
  compact_esc_kernel<<<(unsigned)blocks, 256, 0, s>>>(row_esc, esc_tmp, tmp_off, R, esc, esc_bytes);
  return launched("compact_esc_kernel");
}


namespace bn {

// ---------------------------------------------------------------------------------------------
// Expander that allocates nothing: bn_rice_to_r4_static.
//
// Some hosts of this library cannot call cudaMalloc where they load weights: a plugin running
// inside a framework whose allocator owns the whole device (a second allocator would fragment or
// exhaust it), code that loads layers on a stream while another stream is being captured into a
// CUDA graph (an allocation there is an error), or a service with a fixed memory budget audited at
// start-up. For them the scratch of the two-step expander lives in this fixed device array, which
// every GPU that loads the library holds until the process exits.
// ---------------------------------------------------------------------------------------------
constexpr int64_t STATIC_MAX_ROWS = 65536;              // rows per call
constexpr int64_t STATIC_MAX_WEIGHTS = 16ll << 20;      // R * K per call: escape scratch for the worst case
constexpr size_t STATIC_COUNTERS_AT = 0;                // 8 x uint32, padded to 256 bytes
constexpr size_t STATIC_TMP_OFF_AT = 256;               // uint32 [STATIC_MAX_ROWS]
constexpr size_t STATIC_ESC_AT = STATIC_TMP_OFF_AT + (size_t)STATIC_MAX_ROWS * 4;
constexpr size_t STATIC_BYTES = STATIC_ESC_AT + (size_t)STATIC_MAX_WEIGHTS;  // 16.25 MiB + 256 B

static __device__ __align__(256) unsigned char g_static_scratch[STATIC_BYTES];

// Escape runs -> row order, sizes read on the device: n_esc = counters[2]; at most esc_cap - 1
// escape bytes are written, then the closing 0. info = {n_esc, R - first bad row (0: none),
// 1 if esc_cap was too small (esc is then cut short), 0}.
__global__ void __launch_bounds__(256) compact_esc_static_kernel(const uint32_t *__restrict__ row_esc, const uint8_t *__restrict__ esc_tmp, const uint32_t *__restrict__ tmp_off, const uint32_t *__restrict__ counters, int64_t R, uint8_t *__restrict__ esc, uint64_t esc_cap, uint32_t *__restrict__ info) {
  const uint64_t n_esc = counters[2], room = esc_cap - 1;
  const uint32_t lane = lane_id();
  for (int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); row < R; row += (int64_t)gridDim.x * 8) {
    const uint64_t b = row_esc[row], e = row + 1 < R ? (uint64_t)row_esc[row + 1] : n_esc;
    const uint8_t *src = esc_tmp + tmp_off[row];
    for (uint64_t i = lane; b + i < e && b + i < room; i += 32) esc[b + i] = src[i];
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    esc[n_esc < room ? n_esc : room] = 0;
    info[0] = (uint32_t)n_esc, info[1] = counters[1], info[2] = n_esc > room ? 1u : 0u, info[3] = 0u;
  }
}

// The scratch array's device address on the current device, looked up once per device. The cache
// is atomic: two host threads making their first call together both look the address up and
// store the same value. It does not outlive cudaDeviceReset (the address belongs to the context).
static int static_scratch(unsigned char **out) {
  static std::atomic<unsigned char *> ptr[64];
  int dev = 0;
  BN_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(BN_ERR_ARG, "bn_rice_to_r4_static: device index out of range");
  unsigned char *known = ptr[dev].load(std::memory_order_acquire);
  if (!known) {
    // g_static_scratch names the array on the host side only; kernels need its device address
    void *p = nullptr;
    BN_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
    known = static_cast<unsigned char *>(p);
    ptr[dev].store(known, std::memory_order_release);
  }
  *out = known;
  return BN_OK;
}

}  // namespace bn

extern "C" int bn_rice_to_r4_static(const uint8_t *meta, const uint32_t *bits, uint64_t nwords, const uint32_t *roff, const uint8_t *table, int64_t R, int64_t K, uint16_t *codes, uint8_t *flags, uint32_t *row_esc, uint8_t *esc, uint64_t esc_cap, uint32_t *info, void *stream) {
  using namespace bn;
  if (int e = check_stream(meta, bits, roff, R, K)) return e;
  if (!table || !codes || !flags || !row_esc || !esc || !info || esc_cap < 1) return fail(BN_ERR_ARG, "bn_rice_to_r4_static: null pointer or empty esc");
  if (K % 4) return fail(BN_ERR_ARG, "R4 needs K % 4 == 0");
  if (R > STATIC_MAX_ROWS || K > STATIC_MAX_WEIGHTS / (R > 0 ? R : 1)) return fail(BN_ERR_CAPACITY, "bn_rice_to_r4_static: at most 65536 rows and 16 Mi weights per call (expand larger tensors in row chunks, or use bn_rice_to_r4 with caller scratch)");
  unsigned char *scratch = nullptr;
  if (int e = static_scratch(&scratch)) return e;
  cudaStream_t s = (cudaStream_t)stream;
  uint32_t *counters = reinterpret_cast<uint32_t *>(scratch + STATIC_COUNTERS_AT);
  uint32_t *tmp_off = reinterpret_cast<uint32_t *>(scratch + STATIC_TMP_OFF_AT);
  uint8_t *esc_tmp = scratch + STATIC_ESC_AT;
  // the array keeps the previous call's contents: the counters must start at zero
  BN_CUDA(cudaMemsetAsync(counters, 0, 8 * sizeof(uint32_t), s));
  if (R > 0) {
    RiceArgs a{};
    a.meta = meta, a.bits = bits, a.nwords = nwords, a.roff = roff, a.table = table, a.R = R, a.K = K, a.T = (int)tiles(K);
    a.codes = codes, a.flags = flags, a.row_cnt = row_esc, a.esc_tmp = esc_tmp, a.esc_cap = (uint64_t)STATIC_MAX_WEIGHTS, a.tmp_off = tmp_off, a.counters = counters;
    if (int e = launch_rice_r4(a, s)) return e;
    scan_rows_kernel<<<1, 1024, 0, s>>>(row_esc, R, row_esc);
    if (int e = launched("scan_rows_kernel")) return e;
  }
  int64_t blocks = (R + 7) / 8;
  if (blocks > 2048) blocks = 2048;
  if (blocks < 1) blocks = 1;
  compact_esc_static_kernel<<<(unsigned)blocks, 256, 0, s>>>(row_esc, esc_tmp, tmp_off, counters, R, esc, esc_cap, info);
  return launched("compact_esc_static_kernel");
}

// ---------------------------------------------------------------------------------------------
// Format 1 entry points
// ---------------------------------------------------------------------------------------------
static int f1_grid(int64_t R) {
  const int64_t blocks = (R + 7) / 8;
  return (int)(blocks < 148 * 8 ? blocks : 148 * 8);
}

extern "C" int bn_f1_offsets(const uint8_t *meta, const uint32_t *idx, uint64_t nwords, int64_t R, int64_t K, uint32_t *woff, uint32_t *eoff, uint32_t *scratch, uint32_t *totals, void *stream) {
  if (!meta || !idx || !woff || !eoff || !scratch || !totals || R < 0 || K <= 0) return fail(BN_ERR_ARG, "bn_f1_offsets: null pointer or bad size");
  if (R == 0) return BN_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int T = (int)tiles(K);
  uint32_t *words = scratch, *count = scratch + R;  // scratch: 2 R words
  f1_row_words_kernel<<<f1_grid(R), 256, 0, s>>>(meta, R, T, words);
  if (int e = launched("f1_row_words_kernel")) return e;
  scan_rows_kernel<<<1, 1024, 0, s>>>(words, R, woff);
  if (int e = launched("scan_rows_kernel")) return e;
  f1_row_escapes_kernel<<<f1_grid(R), 256, 0, s>>>(meta, idx, nwords, woff, R, T, count);
  if (int e = launched("f1_row_escapes_kernel")) return e;
  scan_rows_kernel<<<1, 1024, 0, s>>>(count, R, eoff);
  if (int e = launched("scan_rows_kernel")) return e;
  f1_totals_kernel<<<1, 1, 0, s>>>(woff, words, eoff, count, R, totals);
  return launched("f1_totals_kernel");
}

static RiceArgs f1_args(const uint8_t *meta, const uint32_t *idx, uint64_t nwords, const uint32_t *woff, const uint8_t *esc, uint64_t n_esc, const uint32_t *eoff, const uint8_t *table, int64_t R, int64_t K) {
  RiceArgs a{};
  a.meta = meta, a.bits = idx, a.nwords = nwords, a.roff = woff, a.table = table, a.R = R, a.K = K, a.T = (int)tiles(K);
  a.f1_esc = esc, a.f1_nesc = n_esc, a.f1_eoff = eoff;
  return a;
}

static int check_f1(const uint8_t *meta, const uint32_t *idx, const uint32_t *woff, const uint8_t *esc, const uint32_t *eoff, const uint8_t *table, int64_t R, int64_t K) {
  if (!meta || !idx || !woff || !esc || !eoff || !table) return fail(BN_ERR_ARG, "null format-1 array");
  if (R < 0 || K <= 0) return fail(BN_ERR_ARG, "bad matrix size");
  return BN_OK;
}

extern "C" int bn_f1_ranks(const uint8_t *meta, const uint32_t *idx, uint64_t nwords, const uint32_t *woff, const uint8_t *esc, uint64_t n_esc, const uint32_t *eoff, const uint8_t *table, int64_t R, int64_t K, uint8_t *ranks, void *stream) {
  if (int e = check_f1(meta, idx, woff, esc, eoff, table, R, K)) return e;
  if (!ranks) return fail(BN_ERR_ARG, "bn_f1_ranks: null output");
  if (R == 0) return BN_OK;
  RiceArgs a = f1_args(meta, idx, nwords, woff, esc, n_esc, eoff, table, R, K);
  a.ranks = reinterpret_cast<uint32_t *>(ranks), a.rend = nullptr;
  rice_kernel<RICE_RANKS, 1><<<rice_grid(R), RICE_THREADS, 0, (cudaStream_t)stream>>>(a);
  return launched("rice_kernel<ranks, format 1>");
}

extern "C" int bn_f1_unpack(const uint8_t *meta, const uint32_t *idx, uint64_t nwords, const uint32_t *woff, const uint8_t *esc, uint64_t n_esc, const uint32_t *eoff, const uint8_t *table, const uint8_t *raw, int64_t R, int64_t K, uint16_t *out, void *stream) {
  if (int e = check_f1(meta, idx, woff, esc, eoff, table, R, K)) return e;
  if (!raw || !out) return fail(BN_ERR_ARG, "bn_f1_unpack: null pointer");
  if (R == 0) return BN_OK;
  RiceArgs a = f1_args(meta, idx, nwords, woff, esc, n_esc, eoff, table, R, K);
  a.raw = raw, a.out = out, a.rend = nullptr;
  rice_kernel<RICE_UNPACK, 1><<<rice_grid(R), RICE_THREADS, 0, (cudaStream_t)stream>>>(a);
  return launched("rice_kernel<unpack, format 1>");
}

extern "C" int bn_f1_to_r4(const uint8_t *meta, const uint32_t *idx, uint64_t nwords, const uint32_t *woff, const uint8_t *esc, uint64_t n_esc, const uint32_t *eoff, const uint8_t *table, int64_t R, int64_t K, uint16_t *codes, uint8_t *flags, uint32_t *row_cnt, uint8_t *esc_tmp, uint64_t esc_cap, uint32_t *tmp_off, uint32_t *counters, void *stream) {
  if (int e = check_f1(meta, idx, woff, esc, eoff, table, R, K)) return e;
  if (!codes || !flags || !row_cnt || !esc_tmp || !tmp_off || !counters) return fail(BN_ERR_ARG, "bn_f1_to_r4: null output");
  if (K % 4) return fail(BN_ERR_ARG, "R4 needs K % 4 == 0");
  BN_CUDA(cudaMemsetAsync(counters, 0, 8 * sizeof(uint32_t), (cudaStream_t)stream));
  if (R == 0) return BN_OK;
  RiceArgs a = f1_args(meta, idx, nwords, woff, esc, n_esc, eoff, table, R, K);
  a.codes = codes, a.flags = flags, a.row_cnt = row_cnt, a.esc_tmp = esc_tmp, a.esc_cap = esc_cap, a.tmp_off = tmp_off, a.counters = counters;
  rice_kernel<RICE_R4, 1><<<rice_grid(R), RICE_THREADS, 0, (cudaStream_t)stream>>>(a);
  return launched("rice_kernel<r4, format 1>");
}
