/*
 * binade_b200 — C ABI of the B200 (sm_100a) implementation of Binade's data-parallel hot path.
 *
 * Two shared libraries export these symbols:
 *   libbinade_b200.so       the CUDA entry points (section 2); links the CUDA runtime
 *   libbinade_b200_host.so  the host-side codec used by the packer (section 3); no CUDA
 *
 * Conventions
 *   - every entry point returns an int status: BN_OK or a BN_ERR_* code; bn_last_error()
 *     returns a thread-local message for the last non-zero status of the calling thread;
 *   - every pointer of section 2 is a DEVICE pointer owned by the caller (inputs are never
 *     written; outputs must not alias inputs); the library allocates nothing unless stated;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream); calls only
 *     enqueue work and return without synchronising;
 *   - BF16 values travel as uint16_t bit patterns; all integers are little-endian;
 *   - a matrix has R (or N) rows of K weights, T = ceil(K/128) tiles per row.
 *
 * Each declaration cites the interface of the reference project (GuyShafir/binade v0.1.2, paths
 * relative to its root) that it replaces.
 */
#ifndef BINADE_B200_H
#define BINADE_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ 1. status ------------- */
#define BN_OK 0
#define BN_ERR_ARG 1      /* null pointer, K % 4 != 0, size out of range ...                 */
#define BN_ERR_CUDA 2     /* a CUDA runtime call or launch failed; see bn_last_error()       */
#define BN_ERR_CAPACITY 3 /* an output or scratch buffer given by the caller is too small    */
#define BN_ERR_STREAM 4   /* host codec: a Rice stream does not end where its meta says      */

const char *bn_last_error(void);
/* ABI version of the library: major * 100 + minor. */
int bn_abi_version(void);

/* The R4 in-memory layout of one matrix (binade/mlx/r4.py:143-175):
 *   raw     [N*K]      sign<<7 | mantissa of every weight
 *   codes   [N*T*32]   four 4-bit codes per uint16: nibble j of lane word l of tile t is
 *                      min(rank, 15) of weight 128t + 4l + j; padding weights code 0
 *   flags   [N*T]      non-zero iff the tile holds a code 15 (escape)
 *   esc     [n_esc+1]  exponent bytes of the escaped weights, row-major order, one trailing 0
 *   table   [256]      exponent by rank (only entries 0..14 are read by the kernels)
 *   row_esc [N]        number of escapes before each row
 *   n_esc              escapes in `esc` (which holds n_esc + 1 bytes): lets the kernels fetch a
 *                      row's escape bytes ahead of use without reading past the array
 * Not part of the reference's layout, optional (NULL: the kernels use `esc`), derived from the
 * arrays above by bn_r4_esc_columns for the batch-1 kernels:
 *   esc_cols [n_esc+8] the same escape bytes with every row's run reordered by column: first
 *                      the escapes of weights k with (k % 128) / 8 == 0 in row order, then
 *                      those of column 1, ... 15; zero padding behind
 *   col_esc  [N*16]    where column c of row r starts, counted from row_esc[r]
 * With these a thread that owns a column of a row walks its escape bytes with a cursor of its
 * own, instead of the row's threads agreeing on positions with ballots for every flagged tile. */
typedef struct bn_r4 {
  const uint8_t *raw;
  const uint16_t *codes;
  const uint8_t *flags;
  const uint8_t *esc;
  const uint8_t *table;
  const uint32_t *row_esc;
  uint64_t n_esc;
  const uint8_t *esc_cols;   /* optional (both or neither, else NULL): see bn_r4_esc_columns */
  const uint16_t *col_esc;
} bn_r4;

/* ------------------------------------------------------------------ 2. CUDA entry points -- */

/* Rice stream -> 8-bit ranks. Replaces rice_ranks, binade/mlx/cuda_kernels.py:974-995
 * (Metal twin binade/mlx/rice_kernel.py:71-98).
 *   meta [R*T], bits [nwords], roff [R]  ->  ranks [R, T*128] (padding columns 0),
 *   rend [R] = word after the row's last bit; the caller compares it with the next row's roff.
 * Reads of `bits` are clamped to [0, nwords): a corrupt stream cannot read out of bounds. */
int bn_rice_ranks(const uint8_t *meta, const uint32_t *bits, uint64_t nwords, const uint32_t *roff,
                  int64_t R, int64_t K, uint8_t *ranks, uint32_t *rend, void *stream);

/* Rice stream + raw bytes -> BF16 words [R,K], the decode of PackedModel.rows
 * (binade/unpack.py:68-94: rice_ranks, table lookup and bf16.join in one pass). */
int bn_rice_unpack(const uint8_t *meta, const uint32_t *bits, uint64_t nwords, const uint32_t *roff,
                   const uint8_t *table, const uint8_t *raw, int64_t R, int64_t K, uint16_t *out,
                   uint32_t *rend, void *stream);

/* Load-time expander, Rice -> R4, step 1 of 2. Replaces transcode + _rank_chunks
 * (binade/mlx/r4.py:119-175), which decode to 8-bit ranks, re-read them with elementwise ops
 * and gather escapes on the host.
 *   outputs  codes [R*T*32], flags [R*T], row_cnt [R] (escapes of each row)
 *   scratch  esc_tmp [esc_cap] escape bytes, esc_cap < 2^32; each row claims, at tmp_off[r], room
 *            for the most escapes its meta bytes allow (a tile can escape only if
 *            qmax << k | (2^k - 1) >= 15) and writes its escapes there in order;
 *            tmp_off [R]; counters: 8 x uint32, 8-byte aligned, zeroed by the call itself:
 *              [1]    R - (first row whose stream does not end at the next row's roff, or at
 *                     nwords for the last row); 0 = every row ends where it must
 *              [2]    total number of escapes
 *              [4..5] uint64: bytes of esc_tmp claimed
 * When the claimed bytes exceed esc_cap some rows wrote no escape bytes: call again with an
 * esc_tmp of at least that size (codes, flags, row_cnt and counters are complete either way). */
int bn_rice_to_r4(const uint8_t *meta, const uint32_t *bits, uint64_t nwords, const uint32_t *roff,
                  const uint8_t *table, int64_t R, int64_t K, uint16_t *codes, uint8_t *flags,
                  uint32_t *row_cnt, uint8_t *esc_tmp, uint64_t esc_cap, uint32_t *tmp_off,
                  uint32_t *counters, void *stream);

/* Expander step 2: row_esc = exclusive prefix sum of row_cnt (may alias row_cnt), and the
 * escape runs of esc_tmp compacted into row order: esc [n_esc + 1], last byte 0
 * (binade/mlx/r4.py:164-173). esc must hold counters[2] + 1 bytes. */
int bn_r4_finish(const uint32_t *row_cnt, const uint8_t *esc_tmp, const uint32_t *tmp_off, int64_t R,
                 uint32_t *row_esc, uint8_t *esc, uint64_t esc_bytes, void *stream);

/* The whole expander (both steps above) for callers that must not allocate device memory while
 * they load weights: a plugin inside a framework whose own allocator has taken the device, a
 * loader running next to a stream capture (where cudaMalloc is an error), a service whose memory
 * budget is fixed at start-up. This entry point has no counterpart in the reference. It calls no
 * cudaMalloc/cudaFree and no allocating library routine: its scratch is a fixed 16.25 MiB device
 * array inside the library, held by every GPU that loads the library until the process exits.
 *   limits   R <= 65536 rows and R * K <= 16 Mi weights per call (BN_ERR_CAPACITY beyond: expand
 *            a larger tensor in row chunks, or use bn_rice_to_r4 with scratch of your own)
 *   outputs  codes [R*T*32], flags [R*T], row_esc [R], esc [esc_cap] (escape bytes + a closing
 *            0), info: 4 x uint32 on the device = {number of escapes, R - first bad row (0 = every
 *            row ends where it must), 1 if esc_cap < escapes + 1 (esc is then cut short), 0}
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that
 * device current) and keeps it for the life of that device's context (it does not survive
 * cudaDeviceReset); make that first call before any stream capture begins. All calls share the
 * one array and it keeps the last call's contents (the call clears the counters it needs at
 * zero): two calls whose kernels overlap on the GPU, on different streams or from different
 * threads, race; run them one after the other. */
int bn_rice_to_r4_static(const uint8_t *meta, const uint32_t *bits, uint64_t nwords, const uint32_t *roff,
                         const uint8_t *table, int64_t R, int64_t K, uint16_t *codes, uint8_t *flags,
                         uint32_t *row_esc, uint8_t *esc, uint64_t esc_cap, uint32_t *info, void *stream);

/* ---- Rice (format 2) encoder on the device: BF16 words [R,K] in device memory -> the file
 * arrays, bit for bit what binade/rice.py:57-125 (encode_ranks, choose) and the host encoder of
 * this library write. Three calls, two small reads by the host in between (the exponent histogram,
 * from which the host builds the rank table as binade/format.py:34-42 does, and the number of
 * stream words, to size `bits`):
 *   bn_bf16_split_hist    raw [n] = sign << 7 | mantissa of every word, hist [256] = counts of the
 *                         exponent bytes (binade/bf16.py split + the histogram of pack_tensor)
 *   bn_rice_encode_plan   meta [R*T] (k | qmax << 2 per tile, smallest cost, ties to the smaller k),
 *                         row_words [R], roff [R] = exclusive prefix sum, total [1] = words of the
 *                         stream as uint64 (2^32 or more does not fit the format's uint32 offsets)
 *   bn_rice_encode_write  bits [nwords]: every word of every row's stream (rows start on a word)
 * `rank` is the device copy of the 256-entry exponent -> rank table. */
int bn_bf16_split_hist(const uint16_t *w, int64_t n, uint8_t *raw, uint32_t *hist, void *stream);
int bn_rice_encode_plan(const uint16_t *w, const uint8_t *rank, int64_t R, int64_t K, uint8_t *meta,
                        uint32_t *row_words, uint32_t *roff, uint64_t *total, void *stream);
int bn_rice_encode_write(const uint16_t *w, const uint8_t *rank, const uint8_t *meta,
                         const uint32_t *roff, int64_t R, int64_t K, uint32_t *bits, uint64_t nwords,
                         void *stream);

/* Column-ordered escapes of an R4 matrix of N rows (see bn_r4): esc_cols [w->n_esc + 8] (4-byte
 * aligned) and col_esc [N*16] from w's codes, flags, esc and row_esc. K % 16 == 0. The caller
 * stores the two pointers into its bn_r4 afterwards. */
int bn_r4_esc_columns(const bn_r4 *w, int64_t N, int64_t K, uint8_t *esc_cols, uint16_t *col_esc,
                      void *stream);

/* R4 -> dense BF16 [N,K]; output row r is storage row (r / NB) * RS + R0 + r % NB.
 * Replaces r4_decode, binade/mlx/cuda_kernels.py:897-916. */
int bn_r4_decode(const bn_r4 *w, int64_t N, int64_t K, int64_t NB, int64_t RS, int64_t R0,
                 uint16_t *out, void *stream);

/* ---- format 1 (fixed-width codes with escapes, binade/format.py): file arrays meta [R*T]
 * (b | escape << 4), idx (uint32 words, a tile of width b is 4 b words), esc (exponent bytes of
 * the escaped weights, tensor order), table [256]. The format stores no row offsets, so
 * bn_f1_offsets rebuilds them on the device: woff [R] first index word of each row, eoff [R]
 * escapes before each row, totals [2] = (index words, escapes) implied by meta and idx, which the
 * caller compares with the array sizes (the check of format.decode, binade/format.py:128-133).
 * scratch: 2 R uint32. The three decoders then mirror the format-2 ones (same kernels behind
 * them, a different tile front end): 8-bit ranks, BF16 words, R4 arrays (followed by
 * bn_r4_finish). Replace format.decode_tiles (binade/format.py:104-124) and the format-1 branch
 * of _rank_chunks (binade/mlx/r4.py:134-140), which decode on the host CPU with numpy. */
int bn_f1_offsets(const uint8_t *meta, const uint32_t *idx, uint64_t nwords, int64_t R, int64_t K,
                  uint32_t *woff, uint32_t *eoff, uint32_t *scratch, uint32_t *totals, void *stream);
int bn_f1_ranks(const uint8_t *meta, const uint32_t *idx, uint64_t nwords, const uint32_t *woff,
                const uint8_t *esc, uint64_t n_esc, const uint32_t *eoff, const uint8_t *table,
                int64_t R, int64_t K, uint8_t *ranks, void *stream);
int bn_f1_unpack(const uint8_t *meta, const uint32_t *idx, uint64_t nwords, const uint32_t *woff,
                 const uint8_t *esc, uint64_t n_esc, const uint32_t *eoff, const uint8_t *table,
                 const uint8_t *raw, int64_t R, int64_t K, uint16_t *out, void *stream);
int bn_f1_to_r4(const uint8_t *meta, const uint32_t *idx, uint64_t nwords, const uint32_t *woff,
                const uint8_t *esc, uint64_t n_esc, const uint32_t *eoff, const uint8_t *table,
                int64_t R, int64_t K, uint16_t *codes, uint8_t *flags, uint32_t *row_cnt,
                uint8_t *esc_tmp, uint64_t esc_cap, uint32_t *tmp_off, uint32_t *counters,
                void *stream);

/* Fused R4-decode GEMM on the tensor cores for 1 <= M <= 256 input rows (meant for 5 and more):
 * Y [M,N] = X [M,K] . W^T with the weights decoded to BF16 inside the kernel (tcgen05 MMA, fp32
 * accumulators in tensor memory); the weights are read once whatever M. K % 8 == 0, rows of X
 * 16-byte aligned. The sum over K is formed by the tensor core in its own order: outputs agree
 * with an fp32 reference to one BF16 unit in the last place, not bit for bit with bn_r4_rows.
 * Replaces the fused decode GEMM of _R4._cuda_fused, binade/mlx/r4.py:254-268 (r4_gemm,
 * binade/mlx/cuda_kernels.py:640-700, an mma.sync kernel there). */
int bn_r4_mma(const uint16_t *x, int64_t x_stride, const bn_r4 *w, int64_t M, int64_t N, int64_t K,
              uint16_t *y, int64_t y_stride, void *stream);

/* The same product with the K tiles cut into `split` equal slices, each summed from zero in its
 * own tensor-memory accumulator, the slices' fp32 sums added in slice order and rounded once:
 * the order cuBLAS uses on B200 when it splits K (few input rows, long K; measured: split = 2,
 * fp32 partials). With the split cuBLAS picks for a shape (1 where it does not split) the output
 * carries the bits of a BF16 GEMM on the decoded weight. Replaces the split-K mirroring of
 * binade/mlx/cublas_plan.py:84-192 and the reducers binade/mlx/cuda_kernels.py:685-702.
 * ceil(K/128) % split == 0 and split * (M rounded up to 16) <= 512. */
int bn_r4_mma_split(const uint16_t *x, int64_t x_stride, const bn_r4 *w, int64_t M, int64_t N,
                    int64_t K, uint16_t *y, int64_t y_stride, int split, void *stream);

/* Embedding lookup from an R4 table of `rows` rows: out [n,K] row i = BF16 row ids[i]; an id
 * >= rows gives a row of zeros. Replaces R4Embedding.__call__, binade/mlx/r4.py:308-322 (a graph
 * of elementwise array ops there; one kernel here, no host synchronisation either). */
int bn_r4_lookup(const bn_r4 *w, int64_t rows, const uint32_t *ids, int64_t n, int64_t K,
                 uint16_t *out, void *stream);

/* Embedding lookup from a table kept as a Rice stream (about 10.7 bits per weight resident):
 * out [n,K] row i = BF16 row ids[i] of the `rows` x K table (meta [rows*T], roff [rows], raw
 * [rows*K]); an id >= rows gives a row of zeros. Replaces RiceEmbedding.__call__,
 * binade/mlx/r4.py:357-364 (gather of the rows' meta and offsets, then rice_ranks, then the
 * join): the gather, the decode, the table lookup and the join are one pass here. */
int bn_rice_lookup(const uint8_t *meta, const uint32_t *bits, uint64_t nwords, const uint32_t *roff,
                   const uint8_t *table, const uint8_t *raw, int64_t rows, int64_t K,
                   const uint32_t *ids, int64_t n, uint16_t *out, void *stream);

/* Fused R4-decode products Y [M,N] = X [M,K] . W^T for 1 <= M <= 16 input rows, fp32
 * accumulation in a fixed order per output: 32 lanes, lane l owns weights 128t + 4l + j and adds
 * their products (fused multiply-add) for t then j ascending; columns >= K are skipped; lanes
 * combine with strides 16, 8, 4, 2, 1; one round-to-nearest-even to BF16. M = 1 replaces
 * r4_matvec, binade/mlx/cuda_kernels.py:118-130 (same order for K % 128 == 0). The weights are
 * read once whatever M. x_stride / y_stride: elements between rows of X / Y. Any alignment of x
 * is served; the fastest kernels need x and the raw / codes arrays on 16-byte boundaries and
 * K % 16 == 0 (other calls run a plain-load kernel with the same results). */
int bn_r4_rows(const uint16_t *x, int64_t x_stride, const bn_r4 *w, int64_t M, int64_t N, int64_t K,
               uint16_t *y, int64_t y_stride, void *stream);

/* Up to four batch-1 products that share one input, in one launch: y[i] [N[i]] = W[i] . x for
 * `count` matrices of the same K (q, k and v of an attention block; gate and up of an MLP), every
 * output in the documented order of bn_r4_rows and bit-identical to `count` calls of it. The
 * reference launches one r4_matvec per matrix (binade/mlx/cuda_kernels.py:118-130); small
 * matrices are bound by the launch, not by their bytes. w, N, y: host arrays of `count` entries. */
int bn_r4_rows_multi(const uint16_t *x, const bn_r4 *const *w, const int64_t *N, int count, int64_t K,
                     uint16_t *const *y, void *stream);

/* Expert id of a padding slot: bn_r4_gather computes and stores nothing for it (a caller with a
 * fixed number of slots, e.g. under a CUDA graph, marks the unused ones). */
#define BN_NO_EXPERT 0xFFFFFFFFu

/* G independent matvecs (the decode step of a mixture of experts). Slot g multiplies input row
 * xi[g] of x [., K] by storage rows ei[g] * RS + R0 + r, r < n; a slot with ei[g] == BN_NO_EXPERT
 * is skipped (its output row is left untouched). With split == 0 results go to
 * y [G, n]; with 0 < split < n, rows below split go to y [G, split] and the rest to
 * y2 [G, n - split]. Replaces r4_gather, binade/mlx/cuda_kernels.py:133-146. */
int bn_r4_gather(const uint16_t *x, const bn_r4 *w, const uint32_t *xi, const uint32_t *ei, int64_t G,
                 int64_t n, int64_t K, int64_t RS, int64_t R0, int64_t split, uint16_t *y,
                 uint16_t *y2, void *stream);

/* The same products as bn_r4_gather for G slots, grouped by expert so that an expert's rows are
 * read once for all the slots routed to it (prefill / batched decode of an MoE layer; reference:
 * _gather_mm, binade/mlx/r4.py:225-243, which sorts the slots by expert for its gather GEMM).
 * order [G]: slot numbers sorted by expert; seg [E+1]: expert e owns order[seg[e] .. seg[e+1]);
 * xi [G]: input row of each slot; max_per_expert: an upper bound of seg[e+1] - seg[e] (the token
 * count, when a token names an expert at most once). Outputs as bn_r4_gather, row = slot number.
 * Every output keeps the documented summation order: results are bit-identical to bn_r4_gather.
 * Needs K % 16 == 0. */
int bn_r4_gather_grouped(const uint16_t *x, const bn_r4 *w, const uint32_t *xi, const uint32_t *seg,
                         const uint32_t *order, int64_t E, int64_t G, int64_t max_per_expert,
                         int64_t n, int64_t K, int64_t RS, int64_t R0, int64_t split, uint16_t *y,
                         uint16_t *y2, void *stream);

/* All-gather of small slices over NVLink peer memory, one kernel per rank (multi-GPU form of the
 * hook; the reference is single-device, so there is no counterpart). Every rank calls it with
 * 1..4 segments (one per projection): `locals[g]` is this rank's slice of segment g, `bytes[g]`
 * long (a multiple of 16, 16-byte aligned; host arrays of `segments` entries). `peers[r]` is
 * the address, on this GPU, of rank r's symmetric buffer (256 + 2 * area_bytes bytes, zeroed
 * before the first call, mapped on every rank, e.g. by CUDA IPC or a symmetric-memory
 * allocator; area_bytes >= world * sum(bytes), a multiple of 16); `out` is area_bytes of this
 * rank's own device memory; `counter` is a zeroed uint32 in this rank's device memory that
 * belongs to this set of buffers. After the call, in stream order, segment g starts at byte
 * world * (bytes[0] + .. + bytes[g-1]) of `out` and holds the world slices of that segment in
 * rank order. Ranks must make the same sequence of calls; world <= 8; 1..8 segments. Plain peer
 * stores and flags only (no TMA, no multicast). The wait for the peers' flags is bounded by the
 * GPU's nanosecond timer (two seconds, or what bn_set_wait_limit_ns set): a rank whose peer never
 * arrives sets the device status (bits 16..23) and returns with `out` incomplete. */
int bn_push_gather(const void *const *locals, const uint64_t *bytes, int segments,
                   const uint64_t *peers, uint64_t area_bytes, void *out, int rank, int world,
                   uint32_t *counter, void *stream);
/* The same exchange for a stream of its own, beside other kernels (the next products overlap
 * it): three small launches instead of one kernel that holds an SM while its peer is late: the
 * stores and the copy-out as grids of 128-thread blocks that fit on an SM next to this library's
 * largest matvec block, the wait on the peers' flags as a single warp. `counter` points at FOUR
 * zeroed uint32 here (call number, two tickets, the wait's outcome); one set of buffers may mix
 * both forms. */
int bn_push_gather_beside(const void *const *locals, const uint64_t *bytes, int segments,
                          const uint64_t *peers, uint64_t area_bytes, void *out, int rank, int world,
                          uint32_t *counter, void *stream);

/* Device-side status of the calling thread's current device: 0, or non-zero once a kernel of
 * this library gave up a bounded wait or refused a launch whose shared-memory window did not
 * match (its output is then incomplete): bits 0..7 the batch-1 matvec kernels, bits 8..15 the tensor-core GEMM, bits 16..23 the peer exchange. Every wait inside the
 * kernels is bounded, so a lost copy or an absent peer ends in this status instead of a hang.
 * Synchronises with the device. No counterpart in the reference. */
int bn_device_status(int *status);

/* Clears the device status of the current device (after a caller has handled a failure). */
int bn_device_status_reset(void);

/* Bound, in nanoseconds, of every later wait on a peer's flag (bn_push_gather); 0 restores the
 * default of two seconds. Process-wide. No counterpart in the reference. */
int bn_set_wait_limit_ns(uint64_t ns);

/* ------------------------------------------------------------------ 3. host codec --------- */

/* Last error message of the calling thread, for the host codec library. */
const char *bn_host_last_error(void);

/* BF16 words -> raw bytes, exponent histogram (binade/bf16.py:20-33 and the first pass of
 * pack_tensor, binade/pack.py:74-75). hist [256] is ADDED to. raw may be NULL. */
int bn_host_split_hist(const uint16_t *w, int64_t n, uint8_t *raw, int64_t *hist);

/* Histogram -> (table, rank). binade/format.py:34-42. */
int bn_host_rank_table(const int64_t *hist, uint8_t *table, uint8_t *rank);

/* Format-2 (Rice) encoder over rows of BF16 words: binade/rice.py:57-125 fed with
 * rank[bf16.exponent(w)] as pack_tensor does (binade/pack.py:80-83).
 *   w [R*K], rank [256] -> meta [R*T], roff [R], words [cap_words].
 * Returns in *nwords the stream length; when it exceeds cap_words (or words == NULL) nothing is
 * written to `words` and the status is BN_ERR_CAPACITY, so a first call can size the buffer.
 * `threads` <= 0 uses every available core. */
int bn_host_rice_encode(const uint16_t *w, const uint8_t *rank, int64_t R, int64_t K, uint8_t *meta,
                        uint32_t *roff, uint32_t *words, uint64_t cap_words, uint64_t *nwords,
                        int threads);

/* The same encoder fed with ready-made ranks [R*K] (encode_ranks, binade/rice.py:76-119). */
int bn_host_rice_encode_ranks(const uint8_t *ranks, int64_t R, int64_t K, uint8_t *meta, uint32_t *roff,
                              uint32_t *words, uint64_t cap_words, uint64_t *nwords, int threads);

/* Format-1 encoder (binade/format.py:46-101: choose, pack_codes, encode) straight from BF16 words:
 * meta [R*T] = b | 16 (escape mode), idx = the tiles' index words (a tile of width b is 4 b
 * words), esc = exponent bytes of the escaped weights in tensor order. counts[0], counts[1] =
 * words and escapes needed; BN_ERR_CAPACITY when a buffer is smaller (call once with zero
 * capacities to size them). */
int bn_host_f1_encode(const uint16_t *w, const uint8_t *rank, int64_t R, int64_t K, uint8_t *meta,
                      uint32_t *idx, uint64_t cap_idx, uint8_t *esc, uint64_t cap_esc,
                      uint64_t *counts, int threads);

#ifdef __cplusplus
}
#endif
#endif /* BINADE_B200_H */
