// Pieces of the eight-threads-per-row R4 decode shared by the batch-1 matvec and the tensor-core
// GEMM (device only): a thread's private cp.async ring in shared memory, the escape window a
// row's threads hold in registers, and the patch of a tile's escaped weights.
#pragma once

#include "common.cuh"

namespace bn {

// Copies of this thread's bytes of one tile into its slot (R rows per warp: 4R raw bytes and 2R
// code bytes per thread; with R = 1 the even lanes copy the code words of two lanes, cp.async
// moving no less than four bytes). `after`: a value computed from the slot's previous contents,
// so that the copy cannot be issued before those have been read.
template <int R, int U>
__device__ __forceinline__ void copy_tile(uint32_t at, uint32_t to_codes, const uint8_t *raw, const uint8_t *codes, bool code_lane, float after) {
  constexpr int SLOT = 192 * R;
  if constexpr (R == 4) {
    asm volatile("cp.async.cg.shared.global [%0+%1], [%2+%3], 16;  // after %4" ::"r"(at), "n"(U * SLOT), "l"(raw), "n"(U * 128), "f"(after) : "memory");
    asm volatile("cp.async.ca.shared.global [%0+%1], [%2+%3], 8;" ::"r"(at + to_codes), "n"(U * SLOT), "l"(codes), "n"(U * 64) : "memory");
  } else if constexpr (R == 2) {
    asm volatile("cp.async.ca.shared.global [%0+%1], [%2+%3], 8;  // after %4" ::"r"(at), "n"(U * SLOT), "l"(raw), "n"(U * 128), "f"(after) : "memory");
    asm volatile("cp.async.ca.shared.global [%0+%1], [%2+%3], 4;" ::"r"(at + to_codes), "n"(U * SLOT), "l"(codes), "n"(U * 64) : "memory");
  } else {
    asm volatile("cp.async.ca.shared.global [%0+%1], [%2+%3], 4;  // after %4" ::"r"(at), "n"(U * SLOT), "l"(raw), "n"(U * 128), "f"(after) : "memory");
    if (code_lane) asm volatile("cp.async.ca.shared.global [%0+%1], [%2+%3], 4;" ::"r"(at + to_codes), "n"(U * SLOT), "l"(codes), "n"(U * 64) : "memory");
  }
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// Waits until all but the newest N cp.async groups of this thread have landed. The value returned
// is an input of every read of the ring that follows, so none of them can move above the wait.
template <int N>
__device__ __forceinline__ uint32_t cp_wait() {
  uint32_t token;
  asm volatile("cp.async.wait_group %1;\n\tmov.u32 %0, 0;" : "=r"(token) : "n"(N) : "memory");
  return token;
}
// This thread's raw bytes (rr: one word per lane word) and code words (cc: two lane words per
// register) of the tile in slot U of the quad at `at`.
template <int R, int U>
__device__ __forceinline__ void ring_read(uint32_t at, uint32_t to_codes, uint32_t token, uint32_t (&rr)[R], uint32_t (&cc)[(R + 1) / 2]) {
  constexpr int SLOT = 192 * R;
  if constexpr (R == 4) {
    asm("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4+%5];" : "=r"(rr[0]), "=r"(rr[1]), "=r"(rr[2]), "=r"(rr[3]) : "r"(at), "n"(U * SLOT), "r"(token));
    asm("ld.shared.v2.u32 {%0, %1}, [%2+%3];" : "=r"(cc[0]), "=r"(cc[1]) : "r"(at + to_codes), "n"(U * SLOT), "r"(token));
  } else if constexpr (R == 2) {
    asm("ld.shared.v2.u32 {%0, %1}, [%2+%3];" : "=r"(rr[0]), "=r"(rr[1]) : "r"(at), "n"(U * SLOT), "r"(token));
    asm("ld.shared.u32 %0, [%1+%2];" : "=r"(cc[0]) : "r"(at + to_codes), "n"(U * SLOT), "r"(token));
  } else {
    uint16_t c;
    asm("ld.shared.u32 %0, [%1+%2];" : "=r"(rr[0]) : "r"(at), "n"(U * SLOT), "r"(token));
    asm("ld.shared.u16 %0, [%1+%2];" : "=h"(c) : "r"(at + to_codes), "n"(U * SLOT), "r"(token));
    cc[0] = c;
  }
}
// x and the table never change after the block-wide barrier that publishes them; `ready` is a
// value produced after that barrier, so no read can move above it.
__device__ __forceinline__ uint32_t lut_read(uint32_t addr, uint32_t ready) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr), "r"(ready));
  return v;
}
// bit 4j of the result: nibble j of c is 15
__device__ __forceinline__ uint32_t hits15(uint32_t c) {
  const uint32_t t = c & (c >> 1);
  return t & (t >> 2) & 0x11111111u;
}

// Escape bytes of a row's window: word p of the row's threads holds bytes base + 4p .. + 3.
struct EscWindow {
  uint32_t word, base;
};

__device__ __forceinline__ uint32_t window_load(const uint8_t *__restrict__ esc, uint64_t cap, uint32_t off) {
  if ((uint64_t)off + 4 <= cap) return __ldg(reinterpret_cast<const uint32_t *>(esc + off));
  uint32_t v = 0;  // the array's last, partial word: byte by byte
#pragma unroll
  for (int i = 0; i < 4; i++)
    if ((uint64_t)off + i < cap) v |= (uint32_t)__ldg(esc + off + i) << (8 * i);
  return v;
}

// val into pair word k of the four from w[B]
template <int B, int N>
__device__ __forceinline__ void or_into(uint32_t k, uint32_t val, uint32_t (&w)[N]) {
#pragma unroll
  for (int i = 0; i < 4 && B + i < N; i++) w[B + i] |= k == (uint32_t)i ? val : 0u;
}

// Geometry of a warp that walks R rows side by side (R = 4, 2 or 1): 32 / R threads per row, a
// thread plays R consecutive virtual lanes.
template <int R>
struct OctGeom {
  static constexpr int TPR = 32 / R;                  // threads per row
  static constexpr int NC = (R + 1) / 2;              // code registers per thread and tile (two lane words each)
  static constexpr uint32_t SLOT = 192 * R;           // a warp's bytes of one tile: 32 x 4R raw, 32 x 2R codes
  static constexpr uint32_t QUAD = 4 * SLOT;
  static constexpr uint32_t WINDOW = 4 * TPR;         // escape bytes a row's window holds
};

// General case of a flagged tile: some thread holds several escapes. Inclusive scan of the counts
// over the row's threads, then every thread walks its own hits. Whole warp calls it. Inlined:
// as a separate function its call made the caller keep registers in local memory around it, and
// those loads and stores (evicted from L1 by the streamed weights) cost more than the path itself.
template <int R>
__device__ __forceinline__ uint32_t escape_general(uint32_t (&w)[2 * R], uint32_t h0, uint32_t h1, uint32_t epos, uint32_t win_word, uint32_t win_base, const uint8_t *__restrict__ esc, uint32_t lane) {
  using Geo = OctGeom<R>;
  const uint32_t p = lane & (Geo::TPR - 1), cnt = __popc(h0) + __popc(h1);
  uint32_t s = cnt;
#pragma unroll
  for (int d = 1; d < Geo::TPR; d <<= 1) {
    const uint32_t n = __shfl_up_sync(BN_FULL, s, d, Geo::TPR);
    if (p >= (uint32_t)d) s += n;
  }
  const uint32_t tot = __shfl_sync(BN_FULL, s, Geo::TPR - 1, Geo::TPR);
  uint32_t q = epos + s - cnt;
#pragma unroll
  for (int half = 0; half < Geo::NC; half++) {
    uint32_t h = half ? h1 : h0;
    while (__any_sync(BN_FULL, h != 0)) {
      const uint32_t bit = (uint32_t)__ffs((int)h) - 1u;  // 4j
      const uint32_t idx = q - win_base;
      const uint32_t v = __shfl_sync(BN_FULL, win_word, (lane & ~(Geo::TPR - 1)) | ((idx >> 2) & (Geo::TPR - 1)));
      uint32_t e = __byte_perm(v, 0u, 0x4440u | (idx & 3u));
      if (h != 0 && idx >= Geo::WINDOW) e = esc[q];  // outside the window (a row dense with escapes)
      const uint32_t val = e << (7u + ((bit & 4u) << 2));
      if (h != 0) {
        if (half) or_into<4>(bit >> 3, val, w);
        else or_into<0>(bit >> 3, val, w);
        q++;
        h &= h - 1u;
      }
    }
  }
  return tot;
}

// Column-ordered escapes (bn_r4::esc_cols, col_esc): a thread walks the stream of a column it owns
// with a cursor of its own; `word` is the aligned word of esc_cols that holds byte q.
struct EscStream {
  uint32_t q, word;
};
__device__ __forceinline__ void stream_open(EscStream &e, const uint8_t *__restrict__ esc_cols, uint32_t q) {
  e.q = q;
  e.word = __ldg(reinterpret_cast<const uint32_t *>(esc_cols + (q & ~3u)));
}
// Applies the escapes h (bit 4j: weight j of the column's eight in this tile) to the pair words
// w[B .. B+3]. Threads call it on their own (no warp-wide operation inside).
template <int B, int N>
__device__ __forceinline__ void stream_patch(uint32_t h, EscStream &e, const uint8_t *__restrict__ esc_cols, uint32_t (&w)[N]) {
  do {
    const uint32_t bit = (uint32_t)__ffs((int)h) - 1u;
    const uint32_t v = __byte_perm(e.word, 0u, 0x4440u | (e.q & 3u));
    or_into<B>(bit >> 3, v << (7u + ((bit & 4u) << 2)), w);
    e.q++;
    if ((e.q & 3u) == 0) e.word = __ldg(reinterpret_cast<const uint32_t *>(esc_cols + e.q));  // used at the column's next escape at the earliest
    h &= h - 1u;
  } while (h);
}

// What a thread needs to know about itself and its row's matrix while it decodes.
struct OctSelf {
  uint32_t lane, lane_hi, to_codes, lut, ready, gmask, ltg;  // lane_hi: first lane of this thread's row
  const uint8_t *esc;
  uint64_t esc_cap;
  const uint8_t *esc_cols;
};

// Applies a flagged tile's escapes to the pair words w of this thread (cc: its code registers)
// and advances the row's cursor; slides the window on when the cursor is half-way through it.
// Whole warp calls it (a warp takes this path when any of its rows flags the tile).
template <int R>
__device__ __forceinline__ void oct_patch(uint32_t &epos, EscWindow &win, uint32_t (&w)[2 * R], const uint32_t (&cc)[(R + 1) / 2], const OctSelf &me) {
  using Geo = OctGeom<R>;
  uint32_t hits[Geo::NC];
#pragma unroll
  for (int i = 0; i < Geo::NC; i++) hits[i] = hits15(cc[i]);
  const uint32_t upper = Geo::NC > 1 ? hits[Geo::NC - 1] : 0u, h = hits[0] | upper;
  const bool several = ((hits[0] & (hits[0] - 1u)) | (upper & (upper - 1u))) != 0 || (hits[0] != 0 && upper != 0);
  const uint32_t one = __ballot_sync(BN_FULL, h != 0), many = __ballot_sync(BN_FULL, several);
  if (__builtin_expect(many == 0, 1)) {
    // at most one escape per thread (nearly always one in the whole warp): straight-line code.
    // Its byte is as many places after the row's cursor as threads of the row before this one
    // hold an escape; the window reaches that far, since it is slid on as soon as the cursor
    // is half-way through it and a tile adds at most one escape per thread here.
    const uint32_t idx = epos + __popc(one & me.ltg) - win.base;
    const uint32_t v = __shfl_sync(BN_FULL, win.word, me.lane_hi | (idx >> 2));
    const uint32_t e = h ? __byte_perm(v, 0u, 0x4440u | (idx & 3u)) : 0u;  // threads without an escape OR nothing in
    const uint32_t bit = 31u - (uint32_t)__clz((int)h);  // 4j: weight j of the register's eight (h holds one bit)
    const uint32_t val = e << (7u + ((bit & 4u) << 2));
    const uint32_t k = (bit >> 3) & 3u;
    const uint32_t lo = upper ? 0u : val, hi = upper ? val : 0u;
#pragma unroll
    for (int i = 0; i < 4 && i < 2 * R; i++) w[i] |= k == (uint32_t)i ? lo : 0u;
#pragma unroll
    for (int i = 4; i < 2 * R; i++) w[i] |= k == (uint32_t)(i - 4) ? hi : 0u;
    epos += __popc(one & me.gmask);
  } else {
    epos += escape_general<R>(w, hits[0], upper, epos, win.word, win.base, me.esc, me.lane);
  }
  if (__builtin_expect(epos - win.base >= Geo::WINDOW / 2, 0)) {  // slide the window on (the load returns while tiles decode)
    win.base = epos & ~3u;
    win.word = window_load(me.esc, me.esc_cap, win.base + (me.lane & (Geo::TPR - 1)) * 4u);
  }
}

}  // namespace bn
