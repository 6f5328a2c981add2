// Batch-1 fused R4 matvec, eight threads per weight row.
//
// The documented summation order has 32 virtual lanes per output row (lane l owns weights
// 128t + 4l + j of every tile t). Here one thread plays four consecutive virtual lanes, so eight
// threads cover a row and a warp walks four rows side by side:
//
//   thread p of a row's eight   virtual lanes 4p .. 4p+3: 16 consecutive weights of every tile,
//                               i.e. 16 bytes of raw bytes and 8 bytes of code words per tile,
//                               four fp32 accumulators
//   loads                       every thread copies its own bytes into a private ring in shared
//                               memory with cp.async, NQ quads (of four tiles) ahead of the quad
//                               being decoded; groups complete in order, so "all but the newest
//                               NQ - 1" is one wait instruction and costs no registers. The ring
//                               runs on across the warp's rows, so it never drains between rows
//   x                           BF16 in shared memory, multiplied with fma.rn.f32.bf16
//   table                       256-entry pair table (code byte -> two exponents placed in a
//                               BF16x2 word), one column per lane, on a 64 KB boundary of the
//                               shared window so that a lookup address is one byte permute; x
//                               lives in the unused halves of its entries
//   escapes                     a warp takes the patch path for a tile when any of its four rows
//                               flags it; escape bytes come from a 32-byte window of the row's
//                               escapes held in registers (one word per thread)
//   end of a row                virtual lanes combine with strides 16, 8, 4 by three shuffles
//                               per accumulator, strides 2 and 1 inside the thread
//
// A thread reads back only what it copied itself: no barrier after start-up, no flag, no wait on
// another thread. One launch takes up to four matrices that share x (q/k/v, gate/up), or the
// slots of an expert gather. Needs K % 16 == 0, 640 <= K <= 16384 and 16-byte aligned raw /
// codes / x.
#include "common.cuh"
#include "oct.cuh"

namespace bn {
namespace {

constexpr uint32_t OC_BASE_MAX = 2048;    // the dynamic shared window starts below this address
constexpr uint32_t OC_LUT = 65536;        // absolute shared address of the pair table
constexpr uint32_t OC_TOP = 131072;       // the table (and x) end here; rings sit below the table and above this
constexpr uint32_t OC_SMEM_MAX = 227 * 1024 - 256;  // dynamic shared memory a block may ask for (the kernel also has 64 static bytes)

// This thread's 4R values of x for tile U past xs: two BF16x2 words per lane word.
template <int R, int U>
__device__ __forceinline__ void x_read(uint32_t xs, uint32_t ready, uint32_t (&xx)[2 * R]) {
  if constexpr (R == 4) {
    asm("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4+%5];" : "=r"(xx[0]), "=r"(xx[1]), "=r"(xx[2]), "=r"(xx[3]) : "r"(xs), "n"(U * 512), "r"(ready));
    asm("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4+%5];" : "=r"(xx[4]), "=r"(xx[5]), "=r"(xx[6]), "=r"(xx[7]) : "r"(xs), "n"(U * 512 + 256), "r"(ready));
  } else if constexpr (R == 2) {
    asm("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4+%5];" : "=r"(xx[0]), "=r"(xx[1]), "=r"(xx[2]), "=r"(xx[3]) : "r"(xs), "n"(U * 512), "r"(ready));
  } else {
    asm("ld.shared.v2.u32 {%0, %1}, [%2+%3];" : "=r"(xx[0]), "=r"(xx[1]) : "r"(xs), "n"(U * 512), "r"(ready));
  }
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
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

constexpr int OC_MAT = 4;  // matrices that can share one launch (and one x)

struct OctArgs {
  bn_r4 w[OC_MAT];
  uint16_t *y[OC_MAT];
  int64_t N[OC_MAT];        // rows of each matrix (of one expert, for a gather)
  uint32_t groups[OC_MAT];  // row groups (R rows each) of matrix i
  uint32_t bend[OC_MAT];    // blocks (of grid.x) up to and including matrix i: a block serves one matrix, whose table it builds
  int nmat;
  const uint16_t *x;
  int64_t K;
  int T;
  // expert gather (blockIdx.y = slot, one matrix): rows ei[slot] * RS + R0 .. + N[0], input row
  // xi[slot]; outputs y [G, N], or with 0 < split < N: y [G, split] and y2 [G, N - split]
  const uint32_t *xi, *ei;
  int64_t RS, R0, split;
  uint16_t *y2;
  uint32_t smem;  // dynamic shared memory of the launch, bytes
};

__device__ int g_oct_error;  // set when the shared window does not match the launch; read by bn_device_status()

// Where a block's rings sit in the shared window (absolute shared addresses; base = start of the
// dynamic allocation): warps 0 .. in_a-1 below the table, the others above it.
struct OctLayout {
  uint32_t ring_a, in_a, end;
};
__host__ __device__ inline OctLayout oct_layout(uint32_t base, uint32_t warps, uint32_t ring) {
  OctLayout L;
  L.ring_a = (base + 127u) & ~127u;
  L.in_a = (OC_LUT - L.ring_a) / ring;
  if (L.in_a > warps) L.in_a = warps;
  L.end = OC_TOP + (warps - L.in_a) * ring;
  return L;
}

// Per-thread state of the decode side.
template <int R>
struct OctRow {
  float acc[R];
  uint32_t epos;  // the row's escape cursor
  EscWindow win;
  EscStream col[(R + 1) / 2];  // with column-ordered escapes instead: one stream per code register
};

// One tile of this thread's row, decoded: pair words (escapes not yet applied), the matching
// values of x, and the code registers (the patch path looks for code 15 in them).
template <int R>
struct OctTile {
  uint32_t w[2 * R], xx[2 * R], cc[(R + 1) / 2];
};

// Reads slot U of the quad at `at` and x at xs + U * 512, looks the exponents up.
template <int R, int U>
__device__ __forceinline__ void oct_decode(OctTile<R> &t, const OctSelf &me, uint32_t at, uint32_t xs, uint32_t token) {
  uint32_t rr[R];
  ring_read<R, U>(at, me.to_codes, token, rr, t.cc);
  x_read<R, U>(xs, me.ready, t.xx);
#pragma unroll
  for (int i = 0; i < R; i++) {
    const uint32_t c = t.cc[i >> 1];
    t.w[2 * i] = (__byte_perm(rr[i], 0u, 0x1100) & 0x807F807Fu) | lut_read(__byte_perm(c, me.lut, (i & 1) ? 0x7624 : 0x7604), me.ready);
    t.w[2 * i + 1] = (__byte_perm(rr[i], 0u, 0x3322) & 0x807F807Fu) | lut_read(__byte_perm(c, me.lut, (i & 1) ? 0x7634 : 0x7614), me.ready);
  }
}

// Applies the tile's escapes, if any row of the warp has some, and adds its products.
//   flagged  some row of the warp holds a code 15 in this tile (warp-uniform)
//   live     this thread holds weights in the tile (false only in a row's short last tile)
template <int R, bool COLS>
__device__ __forceinline__ void oct_finish(OctRow<R> &s, OctTile<R> &t, const OctSelf &me, bool flagged, bool live) {
  if (flagged) {
    if constexpr (COLS) {
      const uint32_t h0 = hits15(t.cc[0]);
      if (h0) stream_patch<0>(h0, s.col[0], me.esc_cols, t.w);
      if constexpr (R == 4) {
        const uint32_t h1 = hits15(t.cc[1]);
        if (h1) stream_patch<4>(h1, s.col[1], me.esc_cols, t.w);
      }
    } else {
      oct_patch<R>(s.epos, s.win, t.w, t.cc, me);
    }
  }
  if (live) {  // columns >= K are skipped, not added as zeros
#pragma unroll
    for (int i = 0; i < R; i++) s.acc[i] = fma2_bf16(t.w[2 * i + 1], t.xx[2 * i + 1], fma2_bf16(t.w[2 * i], t.xx[2 * i], s.acc[i]));
  }
}

// R: rows a warp walks side by side; NQ: quads of four tiles in flight per thread; MAXW: most
// warps a block may have (bounds the registers). Both sides of the ring move in quads: a quad
// holds up to four consecutive tiles of one row (fewer at the row's end), so slot addresses
// inside a quad are immediates.
template <int R, int NQ, int MAXW, bool COLS>
__global__ void __launch_bounds__(MAXW * 32, 1) r4_oct_kernel(const __grid_constant__ OctArgs a) {
  static_assert(!COLS || R > 1, "a column (eight weights) is owned by one thread only with two or four rows a warp");
  using Geo = OctGeom<R>;
  constexpr uint32_t SLOT = Geo::SLOT, QUAD = Geo::QUAD;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  __shared__ uint32_t s_tab[16];
  const uint32_t lane = lane_id(), warp = threadIdx.x >> 5, grp = lane / Geo::TPR, p = lane & (Geo::TPR - 1);
  const uint32_t W = blockDim.x >> 5;
  const uint32_t base = smem_addr(smem_raw);
  const int64_t K = a.K;
  const int T = a.T;
  // this block's matrix: blocks are dealt out to the matrices of the launch in proportion to
  // their rows, since a block holds one pair table
  int mi = 0;
  uint32_t b0 = 0;
#pragma unroll
  for (int i = 1; i < OC_MAT; i++)
    if (i < a.nmat && blockIdx.x >= a.bend[i - 1]) mi = i, b0 = a.bend[i - 1];
  const bn_r4 mat = a.w[mi];
  const int64_t N = a.N[mi];
  const uint32_t G = a.groups[mi];
  const int64_t slot = blockIdx.y;
  const uint32_t nwarps = (a.bend[mi] - b0) * W, gw = (blockIdx.x - b0) * W + warp;
  if (a.ei && a.ei[slot] == BN_NO_EXPERT) return;  // a padding slot: nothing to compute, nothing stored
  const int64_t row0 = a.ei ? (int64_t)a.ei[slot] * a.RS + a.R0 : 0;  // storage row of output row 0
  const bool partial = (K & 127) != 0;                    // the last tile of a row is short
  const uint32_t pmax = (uint32_t)(K & 127) / (4u * R);   // threads that hold weights in it
  const uint32_t row_codes = (uint32_t)T * 64u;
  const OctLayout L = oct_layout(base, W, NQ * QUAD);
  if (base > OC_BASE_MAX || L.end > base + a.smem) {  // the host sized the window for another layout
    if (threadIdx.x == 0) atomicExch(&g_oct_error, 1);
    return;
  }
  // this warp's ring: NQ quads of four slots; in a slot, a thread's raw bytes at lane * 4R, its
  // code words at 128R + lane * 2R
  const uint32_t ring = (warp < L.in_a ? L.ring_a + warp * (NQ * QUAD) : OC_TOP + (warp - L.in_a) * (NQ * QUAD)) + lane * (4u * R);
  const uint32_t to_codes = 128u * R - lane * (2u * R);  // from this thread's raw address in a slot to its codes
  const bool code_lane = R > 1 || (lane & 1u) == 0;      // R = 1: even lanes copy the code words of two lanes

  // this thread's output row in group g of the matrix (rows past the matrix's end are clamped to
  // its last row when they are read and are not stored)
  auto row_of = [&](uint32_t g) { return (int64_t)g * R + grp; };

  // ---- load side: runs NQ quads ahead of the decode, straight on into the warp's next group
  uint32_t pg = gw;
  int pt = 0;
  bool plive = pg < G;
  const uint8_t *praw = nullptr, *pcode = nullptr;
  uint32_t m_flag = 0, m_epos = 0, m_col = 0;  // next group's first flag byte of this thread, escape cursor, column starts
  auto aim = [&]() {  // point the load side at group pg and fetch its small per-row data
    const int64_t srow = row0 + min(row_of(pg), N - 1);
    praw = mat.raw + srow * K + p * (4u * R);
    pcode = reinterpret_cast<const uint8_t *>(mat.codes) + srow * row_codes + p * (2u * R);
    m_epos = __ldg(mat.row_esc + srow);
    if constexpr (COLS) m_col = R == 4 ? __ldg(reinterpret_cast<const uint32_t *>(mat.col_esc + srow * 16) + p) : (uint32_t)__ldg(mat.col_esc + srow * 16 + p);
    m_flag = p < 8u && (int)p < T ? (uint32_t)__ldg(mat.flags + srow * T + p) : 0u;
  };
  // tiles of the load side's next quad
  auto load_count = [&]() { return plive ? min(4, T - pt) : 0; };
  // the quad's copies are issued: close the cp.async group, move on (into the next group at a row's end)
  auto load_advance = [&](int n) {
    cp_commit();
    praw += n * 128, pcode += n * 64, pt += n;
    if (plive && pt == T) {
      pt = 0, pg += nwarps, plive = pg < G;
      if (plive) aim();
    }
  };
  // any quad, tile by tile (a row's last quad, short tiles)
  auto load_quad_slow = [&](uint32_t at, int n, float after) {
    for (int u = 0; u < n; u++) {
      const bool short_tile = partial && pt + u == T - 1;
      copy_tile<R, 0>(at + u * SLOT, to_codes, (short_tile && p >= pmax ? praw - p * (4u * R) : praw) + u * 128, pcode + u * 64, code_lane, after);  // threads past the row's end copy thread 0's bytes and ignore them
    }
  };

  if (plive) aim();
  uint32_t c_epos = m_epos, c_flag = m_flag, c_col = m_col;  // the first group's, before the load side moves on
#pragma unroll
  for (int q = 0; q < NQ; q++) {
    const int n = load_count();
    load_quad_slow(ring + q * QUAD, n, 0.0f);
    load_advance(n);
  }
  pdl_launch_dependents();

  // ---- x and the pair table into shared memory (whole block)
  {
    pdl_wait();  // x may be the previous kernel's output; the weights above are not
    const uint32_t tab = threadIdx.x < 15 ? (uint32_t)__ldg(mat.table + threadIdx.x) : 0u;  // in flight together with the loads of x below
    // x: a tile's 256 bytes sit in the unused halves of table entries 2t and 2t+1, placed so that
    // the threads of a row cover all banks with each of their reads: with R = 4, thread p reads
    // values 16p .. 16p+7 from the first half and 16p+8 .. 16p+15 from the second, both at byte
    // 16p of the half; with R = 2 or 1 the tile is simply cut in two
    const uint4 *x8 = reinterpret_cast<const uint4 *>(a.x + (a.ei ? (int64_t)a.xi[slot] * K : 0));
    // (four loads in flight per thread: with few warps and a long row, one load per round would
    // put several memory latencies in front of the first product)
    constexpr int XB = 4;
    for (int i0 = threadIdx.x; i0 < T * 16; i0 += blockDim.x * XB) {
      uint4 v[XB];
#pragma unroll
      for (int j = 0; j < XB; j++) {
        const int i = i0 + j * (int)blockDim.x;
        v[j] = i < T * 16 && (int64_t)i * 8 < K ? __ldg(x8 + i) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int j = 0; j < XB; j++) {
        const int i = i0 + j * (int)blockDim.x;
        const uint32_t t = (uint32_t)i >> 4, q = (uint32_t)i & 15u;  // tile, 16-byte piece of the tile
        const uint32_t half = R == 4 ? q & 1u : q >> 3, piece = R == 4 ? q >> 1 : q & 7u;
        if (i < T * 16) *reinterpret_cast<uint4 *>(smem_raw + (OC_LUT - base) + (2u * t + half) * 256u + 128u + piece * 16u) = v[j];
      }
    }
    if (threadIdx.x < 16) s_tab[threadIdx.x] = tab;
    __syncthreads();
    // entry `code` holds table[code & 15] << 7 | table[code >> 4] << 23 in each of its 32 lanes'
    // words: one 16-byte store writes four lanes
    for (uint32_t i = threadIdx.x; i < 256 * 8; i += blockDim.x) {
      const uint32_t code = i >> 3, v = (s_tab[code & 15] << 7) | (s_tab[code >> 4] << 23);
      *reinterpret_cast<uint4 *>(smem_raw + (OC_LUT - base) + code * 256u + (i & 7u) * 16u) = make_uint4(v, v, v, v);
    }
    __syncthreads();
  }
  if (gw >= G) {
    cp_wait<0>();
    return;
  }
  OctSelf me;
  asm volatile("mov.u32 %0, 0;" : "=r"(me.ready)::"memory");  // after the barrier: orders x / table reads
  me.lane = lane, me.lane_hi = lane & ~(Geo::TPR - 1), me.to_codes = to_codes, me.lut = OC_LUT + lane * 4u;
  me.gmask = (R == 1 ? 0xFFFFFFFFu : ((1u << Geo::TPR) - 1u) << (grp * Geo::TPR)), me.ltg = me.gmask & lanemask_lt();
  const uint32_t xs0 = OC_LUT + 128u + (R == 4 ? p * 16u : R == 2 ? (p >> 3) * 256u + (p & 7u) * 16u : (p >> 4) * 256u + (p & 15u) * 8u);

  // ---- decode side
  uint32_t cg = gw;  // group being decoded
  int ct = 0;        // tile of it
  int64_t c_r = row_of(cg);
  const uint8_t *c_flags = nullptr;  // flag bytes of this thread's row
  me.esc = mat.esc, me.esc_cap = mat.n_esc + 1, me.esc_cols = mat.esc_cols;
  uint32_t fm = 0;      // bit u: some row of the warp flags tile (ct & ~7) + u
  uint32_t nflag = 0;   // this thread's flag byte of the next block of eight tiles (threads p < 8)
  uint32_t xs = xs0;
  OctRow<R> s;
  auto begin_group = [&]() {  // c_epos / c_flag hold the group's cursor and first flag bytes
    const int64_t srow = row0 + min(c_r, N - 1);
    c_flags = mat.flags + srow * T;
    s.epos = c_epos;
    nflag = c_flag;
    if constexpr (COLS) {  // this thread's columns: 2p and 2p + 1 (R = 4: both halves of c_col) or p
      stream_open(s.col[0], me.esc_cols, c_epos + (c_col & 0xFFFFu));
      if constexpr (R == 4) stream_open(s.col[1], me.esc_cols, c_epos + (c_col >> 16));
    } else {
      s.win.base = s.epos & ~3u;
      s.win.word = window_load(me.esc, me.esc_cap, s.win.base + p * 4u);
    }
    xs = xs0;
#pragma unroll
    for (int i = 0; i < R; i++) s.acc[i] = 0.0f;
  };
  begin_group();

  // end of a group: combine the 32 virtual lanes (virtual lane = R * p + i: the strides of R and
  // more run across threads, the smaller ones inside the thread), store, move on to the warp's
  // next group. Returns false when there is none.
  auto end_group = [&]() -> bool {
#pragma unroll
    for (int o = Geo::TPR / 2; o >= 1; o >>= 1) {
#pragma unroll
      for (int i = 0; i < R; i++) s.acc[i] = s.acc[i] + __shfl_xor_sync(BN_FULL, s.acc[i], o);
    }
#pragma unroll
    for (int st = R / 2; st >= 1; st >>= 1) {
#pragma unroll
      for (int i = 0; i < st; i++) s.acc[i] = s.acc[i] + s.acc[i + st];
    }
    if (p == 0 && c_r < N) {
      const uint16_t v = f32_to_bf16_bits(s.acc[0]);
      if (a.ei) {
        if (a.split > 0 && c_r >= a.split) a.y2[slot * (N - a.split) + (c_r - a.split)] = v;
        else a.y[0][slot * (a.split > 0 ? a.split : N) + c_r] = v;
      } else {
        a.y[mi][c_r] = v;
      }
    }
    cg += nwarps;
    if (cg >= G) return false;
    ct = 0;
    c_r = row_of(cg);
    c_epos = m_epos, c_flag = m_flag, c_col = m_col;  // fetched when the load side crossed into this group
    begin_group();
    return true;
  };

  uint32_t at = ring;  // quad being decoded (this thread's raw address in its first slot)
  const uint32_t ring_end = ring + NQ * QUAD;
  for (;;) {
    if ((ct & 7) == 0) {  // a new block of eight tiles: fold the flag bytes, fetch the next block's
      const uint32_t v = __ballot_sync(BN_FULL, nflag != 0);
      fm = (R == 4 ? v | (v >> 8) | (v >> 16) | (v >> 24) : R == 2 ? v | (v >> 16) : v) & 0xFFu;
      const int nt = ct + 8 + (int)p;
      nflag = p < 8u && nt < T ? (uint32_t)__ldg(c_flags + nt) : 0u;
    }
    const uint32_t fq = fm >> (ct & 4);  // bit u: tile ct + u is flagged
    const int cn = min(4, T - ct), pn = load_count();
    const uint32_t token = cp_wait<NQ - 1>();  // all but the newest NQ - 1 groups have landed: this quad's has
    if (R == 1) __syncwarp();                  // a lane reads code words its neighbour copied
    if (cn == 4 && !partial) {
      // four whole tiles; each slot is refilled, with a tile of the quad NQ ahead, once the quad
      // is read
      OctTile<R> t;
      oct_decode<R, 0>(t, me, at, xs, token), oct_finish<R, COLS>(s, t, me, fq & 1u, true);
      oct_decode<R, 1>(t, me, at, xs, token), oct_finish<R, COLS>(s, t, me, fq & 2u, true);
      oct_decode<R, 2>(t, me, at, xs, token), oct_finish<R, COLS>(s, t, me, fq & 4u, true);
      oct_decode<R, 3>(t, me, at, xs, token), oct_finish<R, COLS>(s, t, me, fq & 8u, true);
      if (R == 1) __syncwarp();  // the neighbour's reads too
      if (pn > 0) copy_tile<R, 0>(at, to_codes, praw, pcode, code_lane, s.acc[0]);
      if (pn > 1) copy_tile<R, 1>(at, to_codes, praw, pcode, code_lane, s.acc[0]);
      if (pn > 2) copy_tile<R, 2>(at, to_codes, praw, pcode, code_lane, s.acc[0]);
      if (pn > 3) copy_tile<R, 3>(at, to_codes, praw, pcode, code_lane, s.acc[0]);
    } else {
      for (int u = 0; u < cn; u++) {
        const bool live = !(partial && ct + u == T - 1) || p < pmax;
        OctTile<R> t;
        oct_decode<R, 0>(t, me, at + u * SLOT, xs + u * 512u, token);
        oct_finish<R, COLS>(s, t, me, (fq >> u) & 1u, live);
      }
      if (R == 1) __syncwarp();
      load_quad_slow(at, pn, s.acc[0]);
    }
    load_advance(pn);
    xs += cn * 512u;
    at = at + QUAD == ring_end ? ring : at + QUAD;
    ct += cn;
    if (ct == T) {
      if (!end_group()) break;
    }
  }
  cp_wait<0>();
}

int oct_sms() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

// Dynamic shared memory a block of `warps` warps with rings of `ring` bytes needs, whatever the
// window's start (the kernel re-derives the layout from the real start); 0 if it does not fit.
uint32_t oct_smem(uint32_t warps, uint32_t ring) {
  const uint32_t a = oct_layout(0, warps, ring).end, b = oct_layout(OC_BASE_MAX, warps, ring).end;
  const uint32_t need = a > b ? a : b;  // the window ends at base + smem >= smem
  return need <= OC_SMEM_MAX ? need : 0;
}

template <int R, int NQ, int MAXW, bool COLS>
int launch_oct_with(OctArgs a, unsigned blocks, unsigned slots, unsigned warps, cudaStream_t s) {
  auto kern = r4_oct_kernel<R, NQ, MAXW, COLS>;
  a.smem = oct_smem(warps, NQ * OctGeom<R>::QUAD);
  if (!a.smem || warps > MAXW || NQ * 4 >= a.T) return -1;  // the ring must be shorter than a row (see the kernel's load side)
  BN_CUDA(allow_smem(kern, OC_SMEM_MAX));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(blocks, slots), cfg.blockDim = dim3(warps * 32), cfg.dynamicSmemBytes = a.smem, cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;  // start-up and the first weight loads overlap the previous kernel's tail
  cfg.attrs = attr, cfg.numAttrs = 1;
  BN_CUDA(cudaLaunchKernelEx(&cfg, kern, a));
  return launched("r4_oct_kernel");
}

// The variant for column-ordered escapes when every matrix of the launch carries them.
template <int R, int NQ, int MAXW>
int launch_oct_as(const OctArgs &a, unsigned blocks, unsigned slots, unsigned warps, cudaStream_t s) {
  if constexpr (R > 1) {
    bool cols = true;
    for (int i = 0; i < a.nmat; i++) cols = cols && a.w[i].esc_cols && a.w[i].col_esc;
    if (cols) return launch_oct_with<R, NQ, MAXW, true>(a, blocks, slots, warps, s);
  }
  return launch_oct_with<R, NQ, MAXW, false>(a, blocks, slots, warps, s);
}

// Rows a warp walks side by side for `rows` output rows spread over `blocks` blocks: four when
// that still gives every SM a dozen warps or more, else two, else one (measured on 3840-wide
// rows: 15360 and 8192 rows are fastest with four, 4096 and 2048 with two).
int oct_rows_per_warp(int64_t rows, int64_t blocks) {
  return rows >= blocks * 52 ? 4 : rows >= blocks * 13 ? 2 : 1;
}

}  // namespace

int oct_status(int *status) {
  BN_CUDA(cudaMemcpyFromSymbol(status, g_oct_error, sizeof(int)));
  return BN_OK;
}

int oct_status_reset() {
  const int zero = 0;
  BN_CUDA(cudaMemcpyToSymbol(g_oct_error, &zero, sizeof(int)));
  return BN_OK;
}

// Launch shape: one block per SM (per slot share of the SMs for a gather), dealt out to the
// matrices in proportion to their rows; as many warps as spread a matrix's row groups evenly over
// its blocks; deeper rings when the warps are few, since then they are all the memory
// parallelism there is.
// Fills the launch's shape for R rows per warp: row groups, blocks per matrix (proportional to
// its groups, at least one, summing to `blocks`, which shrinks to the group count when that is
// smaller). Returns the warps a block needs, or -1 when there are fewer blocks than matrices.
static int64_t oct_shape(OctArgs &a, int R, int64_t &blocks) {
  int64_t groups = 0;
  for (int i = 0; i < a.nmat; i++) a.groups[i] = (uint32_t)((a.N[i] + R - 1) / R), groups += a.groups[i];
  if (blocks > groups) blocks = groups;
  if (blocks < a.nmat) return -1;
  int64_t share[OC_MAT], given = 0;
  for (int i = 0; i < a.nmat; i++) share[i] = max((int64_t)1, blocks * a.groups[i] / groups), given += share[i];
  for (int i = 0; given != blocks; i = (i + 1) % a.nmat) {
    if (given < blocks) share[i]++, given++;
    else if (share[i] > 1) share[i]--, given--;
  }
  int64_t warps = 1;
  uint32_t b = 0;
  for (int i = 0; i < OC_MAT; i++) {
    if (i < a.nmat) {
      b += (uint32_t)share[i];
      const int64_t rounds = (a.groups[i] + share[i] * 32 - 1) / (share[i] * 32);
      warps = max(warps, (int64_t)((a.groups[i] + share[i] * rounds - 1) / (share[i] * rounds)));
    }
    a.bend[i] = b;
  }
  return warps;
}

template <int R>
static int oct_launch_r(OctArgs &a, int64_t blocks, int64_t slots, cudaStream_t s) {
  const int64_t warps = oct_shape(a, R, blocks);
  if (warps < 0) return -1;
  int e = -1;
  if (R == 4) {
    if (warps <= 16 && e == -1) e = launch_oct_as<4, 2, 16>(a, (unsigned)blocks, (unsigned)slots, (unsigned)warps, s);
    if (warps <= 26 && e == -1) e = launch_oct_as<4, 1, 26>(a, (unsigned)blocks, (unsigned)slots, (unsigned)warps, s);
    if (e == -1) e = launch_oct_as<4, 1, 32>(a, (unsigned)blocks, (unsigned)slots, (unsigned)warps, s);
  } else if (R == 2) {
    if (warps <= 16 && e == -1) e = launch_oct_as<2, 4, 16>(a, (unsigned)blocks, (unsigned)slots, (unsigned)warps, s);
    if (e == -1) e = launch_oct_as<2, 2, 32>(a, (unsigned)blocks, (unsigned)slots, (unsigned)warps, s);
    if (e == -1) e = launch_oct_as<2, 1, 32>(a, (unsigned)blocks, (unsigned)slots, (unsigned)warps, s);
  } else {
    e = launch_oct_as<1, 2, 32>(a, (unsigned)blocks, (unsigned)slots, (unsigned)warps, s);
    if (e == -1) e = launch_oct_as<1, 1, 32>(a, (unsigned)blocks, (unsigned)slots, (unsigned)warps, s);
  }
  return e;
}

static int oct_launch(OctArgs &a, int64_t slots, cudaStream_t s) {
  const int64_t blocks = (oct_sms() + slots - 1) / slots;
  int64_t rows = 0;
  for (int i = 0; i < a.nmat; i++) rows += a.N[i];
  const int R = oct_rows_per_warp(rows, blocks);
  return R == 4 ? oct_launch_r<4>(a, blocks, slots, s) : R == 2 ? oct_launch_r<2>(a, blocks, slots, s) : oct_launch_r<1>(a, blocks, slots, s);
}

static bool oct_aligned(const bn_r4 *w, const uint16_t *x) {
  return ((reinterpret_cast<uintptr_t>(w->raw) | reinterpret_cast<uintptr_t>(w->codes) | reinterpret_cast<uintptr_t>(x)) & 15) == 0 && ((reinterpret_cast<uintptr_t>(w->esc) | reinterpret_cast<uintptr_t>(w->esc_cols) | reinterpret_cast<uintptr_t>(w->col_esc)) & 3) == 0;
}

// Up to four matrices of the same K against one x; -1 when the shape is outside the kernel's coverage.
int oct_matvec_multi(const bn_r4 *const *w, const int64_t *N, uint16_t *const *y, int nmat, const uint16_t *x, int64_t K, cudaStream_t s) {
  if (nmat < 1 || nmat > OC_MAT || K % 16 || K < 640 || K > 16384) return -1;
  OctArgs a{};
  for (int i = 0; i < nmat; i++) {
    if (N[i] < 1 || N[i] > (1ll << 30) || !oct_aligned(w[i], x)) return -1;
    a.w[i] = *w[i], a.y[i] = y[i], a.N[i] = N[i];
  }
  a.nmat = nmat, a.x = x, a.K = K, a.T = (int)tiles(K);
  return oct_launch(a, 1, s);
}

int oct_matvec(const bn_r4 *w, const uint16_t *x, int64_t N, int64_t K, uint16_t *y, cudaStream_t s) {
  return oct_matvec_multi(&w, &N, &y, 1, x, K, s);
}

int oct_gather(const bn_r4 *w, const uint16_t *x, const uint32_t *xi, const uint32_t *ei, int64_t G, int64_t n, int64_t K, int64_t RS, int64_t R0, int64_t split, uint16_t *y, uint16_t *y2, cudaStream_t s) {
  if (K % 16 || K < 640 || K > 16384 || n < 1 || n > (1ll << 30) || G < 1 || G > 65535 || !oct_aligned(w, x)) return -1;
  OctArgs a{};
  a.w[0] = *w, a.y[0] = y, a.N[0] = n, a.nmat = 1;
  a.x = x, a.K = K, a.T = (int)tiles(K);
  a.xi = xi, a.ei = ei, a.RS = RS, a.R0 = R0, a.split = split, a.y2 = y2;
  return oct_launch(a, G, s);
}

}  // namespace bn
