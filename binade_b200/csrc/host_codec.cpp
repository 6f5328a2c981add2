// Host side of the packer: BF16 split + histogram, rank table, and the format-2 (Rice)
// encoder, multi-threaded over rows. Plain C++17, no CUDA: the packer runs on the host by
// design (the compressed file is what travels to the GPU).
#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstring>
#include <numeric>
#include <thread>
#include <vector>

#include "../../include/binade_b200.h"

namespace {

constexpr int TILE = 128;
thread_local char g_error[256] = "";

int fail(int code, const char *msg) {
  std::snprintf(g_error, sizeof g_error, "%s", msg);
  return code;
}

int pick_threads(int threads, int64_t items) {
  int n = threads > 0 ? threads : (int)std::thread::hardware_concurrency();
  if (n < 1) n = 1;
  if (items < n) n = (int)std::max<int64_t>(1, items);
  return n;
}

// Cost in bits of a tile under parameter k, and its largest quotient.
inline int64_t tile_cost(const uint8_t *r, int n, int k, int *qmax_out) {
  int qmax = 0;
  for (int i = 0; i < n; i++) qmax = std::max(qmax, r[i] >> k);
  int64_t bits = (int64_t)k * n;
  for (int i = 0; i < n; i++) bits += std::min((r[i] >> k) + 1, qmax);
  *qmax_out = qmax;
  return bits;
}

// Smallest-cost k in 0..3 (ties to the smaller k); a k whose qmax exceeds 63 is not allowed.
// k = 0 is kept only when no k is allowed, which cannot happen for 8-bit ranks (255 >> 2 = 63).
inline void choose(const uint8_t *r, int n, int *k_out, int *qmax_out, int64_t *bits_out) {
  int best_k = 0, best_q = 0;
  int64_t best = INT64_MAX;
  for (int k = 0; k <= 3; k++) {
    int q;
    int64_t b = tile_cost(r, n, k, &q);
    if (q > 63) b = INT64_MAX;
    if (k == 0 || b < best) best_k = k, best_q = q, best = b;
  }
  *k_out = best_k, *qmax_out = best_q, *bits_out = best;
}

// Appends bits LSB first into 32-bit words through a 64-bit accumulator.
struct BitWriter {
  uint32_t *words;
  uint64_t acc = 0;
  int fill = 0;
  explicit BitWriter(uint32_t *w) : words(w) {}
  inline void put(uint32_t v, int n) {  // n <= 32
    acc |= (uint64_t)v << fill;
    fill += n;
    if (fill >= 32) {
      *words++ = (uint32_t)acc;
      acc >>= 32;
      fill -= 32;
    }
  }
  inline void flush() {
    if (fill > 0) *words++ = (uint32_t)acc;
    acc = 0, fill = 0;
  }
};

void encode_tile(const uint8_t *r, int n, int k, int qmax, BitWriter &out) {
  if (k) {
    const uint32_t mask = (1u << k) - 1u;
    for (int i = 0; i < n; i++) out.put(r[i] & mask, k);
  }
  uint8_t q[TILE];
  for (int i = 0; i < n; i++) q[i] = (uint8_t)(r[i] >> k);
  for (int j = 0; j < qmax; j++)
    for (int i = 0; i < n; i++)
      if (q[i] >= j) out.put(q[i] > j ? 1u : 0u, 1);
}

}  // namespace

extern "C" const char *bn_host_last_error(void) { return g_error; }

extern "C" int bn_host_split_hist(const uint16_t *w, int64_t n, uint8_t *raw, int64_t *hist) {
  if (!w || !hist || n < 0) return fail(BN_ERR_ARG, "bn_host_split_hist: null pointer");
  int64_t h[256] = {0};
  for (int64_t i = 0; i < n; i++) {
    const uint16_t u = w[i];
    h[(u >> 7) & 0xFF]++;
    if (raw) raw[i] = (uint8_t)(((u >> 8) & 0x80) | (u & 0x7F));
  }
  for (int e = 0; e < 256; e++) hist[e] += h[e];
  return BN_OK;
}

extern "C" int bn_host_rank_table(const int64_t *hist, uint8_t *table, uint8_t *rank) {
  if (!hist || !table || !rank) return fail(BN_ERR_ARG, "bn_host_rank_table: null pointer");
  int order[256];
  std::iota(order, order + 256, 0);
  std::stable_sort(order, order + 256, [&](int a, int b) { return hist[a] > hist[b]; });
  for (int r = 0; r < 256; r++) {
    table[r] = hist[order[r]] > 0 ? (uint8_t)order[r] : 0;
    rank[order[r]] = (uint8_t)r;
  }
  return BN_OK;
}

namespace {

// Rows of ranks come either ready-made (uint8) or from BF16 words through the rank table.
struct RankRows {
  const uint8_t *ranks;
  const uint16_t *w;
  const uint8_t *rank;
  inline void tile(int64_t off, int n, uint8_t *r) const {
    if (ranks) {
      std::memcpy(r, ranks + off, (size_t)n);
    } else {
      for (int i = 0; i < n; i++) r[i] = rank[(w[off + i] >> 7) & 0xFF];
    }
  }
};

int encode_rows(const RankRows &src, int64_t R, int64_t K, uint8_t *meta, uint32_t *roff, uint32_t *words, uint64_t cap_words, uint64_t *nwords, int threads) {
  const int64_t T = (K + TILE - 1) / TILE;
  const int nt = pick_threads(threads, R);
  std::vector<uint64_t> row_words((size_t)R);
  auto run = [&](auto &&fn) {
    std::vector<std::thread> pool;
    const int64_t per = (R + nt - 1) / nt;
    for (int i = 0; i < nt; i++) {
      const int64_t r0 = std::min<int64_t>(R, i * per), r1 = std::min<int64_t>(R, r0 + per);
      if (r0 < r1) pool.emplace_back(fn, r0, r1);
    }
    for (auto &t : pool) t.join();
  };
  // pass 1: per tile k and qmax, per row word count
  run([&](int64_t r0, int64_t r1) {
    uint8_t r[TILE];
    for (int64_t row = r0; row < r1; row++) {
      int64_t bits = 0;
      for (int64_t t = 0; t < T; t++) {
        const int n = (int)std::min<int64_t>(TILE, K - t * TILE);
        src.tile(row * K + t * TILE, n, r);
        int k, qmax;
        int64_t b;
        choose(r, n, &k, &qmax, &b);
        meta[row * T + t] = (uint8_t)(k | (qmax << 2));
        bits += b;
      }
      row_words[(size_t)row] = (uint64_t)((bits + 31) >> 5);
    }
  });
  uint64_t total = 0;
  std::vector<uint64_t> start((size_t)R);
  for (int64_t row = 0; row < R; row++) start[(size_t)row] = total, total += row_words[(size_t)row];
  *nwords = total;
  if (total >= (1ull << 32)) return fail(BN_ERR_CAPACITY, "Rice stream overflows uint32 row offsets");
  for (int64_t row = 0; row < R; row++) roff[row] = (uint32_t)start[(size_t)row];
  if (!words || total > cap_words) return fail(BN_ERR_CAPACITY, "words buffer too small (size it from *nwords)");
  // pass 2: emit each row at its word offset
  run([&](int64_t r0, int64_t r1) {
    uint8_t r[TILE];
    for (int64_t row = r0; row < r1; row++) {
      BitWriter out(words + start[(size_t)row]);
      for (int64_t t = 0; t < T; t++) {
        const int n = (int)std::min<int64_t>(TILE, K - t * TILE);
        src.tile(row * K + t * TILE, n, r);
        const uint8_t m = meta[row * T + t];
        encode_tile(r, n, m & 3, m >> 2, out);
      }
      out.flush();
    }
  });
  return BN_OK;
}


// ---------------------------------------------------------------------------------------------
// Format 1 (binade/format.py): fixed-width codes with escapes. A tile of 128 ranks (rows padded
// with rank 0) is stored with b bits per code in exactly 4 b words, code i at bits i b .., LSB
// first; in escape mode the code 2^b - 1 stands for "next byte of the escape stream", which holds
// the weight's exponent. meta = b | 16 (escape mode). The width is the cheapest of: fixed
// (b = bit length of the largest rank, 128 b bits) and escape widths 1..4 (128 b + 8 per escaped
// weight); ties go to fixed, then to the smaller escape width (binade/format.py:46-60).
// ---------------------------------------------------------------------------------------------
inline void f1_choose(const uint8_t *r, int *b_out, bool *esc_out) {
  int rmax = 0;
  for (int i = 0; i < TILE; i++) rmax = std::max(rmax, (int)r[i]);
  int fixed_b = 0;
  while ((1 << fixed_b) <= rmax) fixed_b++;
  int64_t best = (int64_t)TILE * fixed_b;
  int b = fixed_b;
  bool esc = false;
  for (int w = 1; w <= 4; w++) {
    int over = 0;
    for (int i = 0; i < TILE; i++) over += r[i] >= (1 << w) - 1;
    const int64_t c = (int64_t)TILE * w + 8 * over;
    if (c < best) best = c, b = w, esc = true;
  }
  *b_out = b, *esc_out = esc;
}

int f1_encode(const uint16_t *w, const uint8_t *rank, int64_t R, int64_t K, uint8_t *meta, uint32_t *idx, uint64_t cap_idx, uint8_t *esc, uint64_t cap_esc, uint64_t *counts, int threads) {
  const int64_t T = (K + TILE - 1) / TILE;
  const int nt = pick_threads(threads, R);
  std::vector<uint64_t> row_words((size_t)R), row_esc((size_t)R);
  auto run = [&](auto &&fn) {
    std::vector<std::thread> pool;
    const int64_t per = (R + nt - 1) / nt;
    for (int i = 0; i < nt; i++) {
      const int64_t r0 = std::min<int64_t>(R, i * per), r1 = std::min<int64_t>(R, r0 + per);
      if (r0 < r1) pool.emplace_back(fn, r0, r1);
    }
    for (auto &t : pool) t.join();
  };
  auto tile_ranks = [&](int64_t row, int64_t t, uint8_t *r) {
    const int n = (int)std::min<int64_t>(TILE, K - t * TILE);
    const uint16_t *src = w + row * K + t * TILE;
    for (int i = 0; i < n; i++) r[i] = rank[(src[i] >> 7) & 0xFF];
    for (int i = n; i < TILE; i++) r[i] = 0;  // padding: the most common exponent
    return n;
  };
  // pass 1: widths, and how many words and escapes each row takes
  run([&](int64_t r0, int64_t r1) {
    uint8_t r[TILE];
    for (int64_t row = r0; row < r1; row++) {
      uint64_t words = 0, escapes = 0;
      for (int64_t t = 0; t < T; t++) {
        tile_ranks(row, t, r);
        int b;
        bool em;
        f1_choose(r, &b, &em);
        meta[row * T + t] = (uint8_t)(b | (em ? 16 : 0));
        words += 4 * (uint64_t)b;
        if (em)
          for (int i = 0; i < TILE; i++) escapes += r[i] >= (1 << b) - 1;
      }
      row_words[(size_t)row] = words, row_esc[(size_t)row] = escapes;
    }
  });
  uint64_t nw = 0, ne = 0;
  std::vector<uint64_t> w_at((size_t)R), e_at((size_t)R);
  for (int64_t row = 0; row < R; row++) w_at[(size_t)row] = nw, e_at[(size_t)row] = ne, nw += row_words[(size_t)row], ne += row_esc[(size_t)row];
  counts[0] = nw, counts[1] = ne;
  if ((nw && !idx) || nw > cap_idx || (ne && !esc) || ne > cap_esc) return fail(BN_ERR_CAPACITY, "format-1 buffers too small (size them from counts)");
  // pass 2: the index words and the escape bytes, every row at its own place
  run([&](int64_t r0, int64_t r1) {
    uint8_t r[TILE];
    for (int64_t row = r0; row < r1; row++) {
      uint32_t *out = idx + w_at[(size_t)row];
      uint8_t *eout = esc + e_at[(size_t)row];
      for (int64_t t = 0; t < T; t++) {
        const int n = tile_ranks(row, t, r);
        const uint8_t m = meta[row * T + t];
        const int b = m & 15;
        const bool em = (m & 16) != 0;
        const int cmax = (1 << b) - 1;
        uint64_t acc = 0;
        int fill = 0;
        for (int i = 0; i < TILE; i++) {
          int code = r[i];
          if (em && code >= cmax) {
            code = cmax;
            *eout++ = (uint8_t)(i < n ? (w[row * K + t * TILE + i] >> 7) & 0xFF : 0);  // (padding never escapes: its rank is 0 and cmax >= 1)
          }
          acc |= (uint64_t)code << fill, fill += b;
          if (fill >= 32) *out++ = (uint32_t)acc, acc >>= 32, fill -= 32;
        }
      }
    }
  });
  return BN_OK;
}

}  // namespace

extern "C" int bn_host_rice_encode(const uint16_t *w, const uint8_t *rank, int64_t R, int64_t K, uint8_t *meta, uint32_t *roff, uint32_t *words, uint64_t cap_words, uint64_t *nwords, int threads) {
  if (!w || !rank || !meta || !roff || !nwords || R < 0 || K <= 0) return fail(BN_ERR_ARG, "bn_host_rice_encode: null pointer or bad size");
  return encode_rows(RankRows{nullptr, w, rank}, R, K, meta, roff, words, cap_words, nwords, threads);
}

extern "C" int bn_host_rice_encode_ranks(const uint8_t *ranks, int64_t R, int64_t K, uint8_t *meta, uint32_t *roff, uint32_t *words, uint64_t cap_words, uint64_t *nwords, int threads) {
  if (!ranks || !meta || !roff || !nwords || R < 0 || K <= 0) return fail(BN_ERR_ARG, "bn_host_rice_encode_ranks: null pointer or bad size");
  return encode_rows(RankRows{ranks, nullptr, nullptr}, R, K, meta, roff, words, cap_words, nwords, threads);
}

extern "C" int bn_host_f1_encode(const uint16_t *w, const uint8_t *rank, int64_t R, int64_t K, uint8_t *meta, uint32_t *idx, uint64_t cap_idx, uint8_t *esc, uint64_t cap_esc, uint64_t *counts, int threads) {
  if (!w || !rank || !meta || !counts || R < 0 || K <= 0) return fail(BN_ERR_ARG, "bn_host_f1_encode: null pointer or bad size");
  return f1_encode(w, rank, R, K, meta, idx, cap_idx, esc, cap_esc, counts, threads);
}
