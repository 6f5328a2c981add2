"""TEST INFRASTRUCTURE ONLY: the CPU oracle of the Binade hot path.

Two independent restatements of the reference's algorithms (GuyShafir/binade v0.1.2):

* `np_*` functions: numpy, written for clarity, used on small cases;
* `c_*` functions: ctypes bindings of `binade_oracle.c` (scalar C loops, OpenMP over rows),
  fast enough for the benchmark's full-size matrices and for the timed CPU baseline.

Both are pinned by the golden vectors under tests/golden (made by running the reference's own
numpy code) and by the reference's hand-computed stream (tests/test_rice.py:50-56).
Only tests, the smoke check and the benchmark's CPU-baseline leg may import this module; the
shipped package never does.
"""

from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

TILE = 128  # binade/format.py:17
KMAX, QMAX = 3, 63  # binade/rice.py:29-30
HERE = Path(__file__).resolve().parent
LIB = HERE / "_build" / "libbinade_oracle.so"


# ----------------------------------------------------------------------------- numpy
def np_split(w: np.ndarray):
    """binade/bf16.py:20-33: uint16 BF16 words -> (raw = sign<<7 | mantissa, exponent)."""
    w = w.astype(np.uint16)
    return (((w >> 8) & 0x80) | (w & 0x7F)).astype(np.uint8), ((w >> 7) & 0xFF).astype(np.uint8)


def np_join(raw: np.ndarray, exps: np.ndarray) -> np.ndarray:
    """binade/bf16.py:36-41."""
    r, e = raw.astype(np.uint16), exps.astype(np.uint16)
    return ((r & 0x80) << 8) | (e << 7) | (r & 0x7F)


def np_rank_table(hist: np.ndarray):
    """binade/format.py:34-42: descending count, ties to the smaller exponent; table entries of
    absent exponents are 0."""
    order = sorted(range(256), key=lambda e: (-int(hist[e]), e))
    table = np.array([e if hist[e] > 0 else 0 for e in order], np.uint8)
    rank = np.zeros(256, np.uint8)
    rank[order] = np.arange(256, dtype=np.uint8)
    return table, rank


def _tile_view(ranks: np.ndarray):
    """[R,K] -> ([R*T,128] int64 zero padded, [R*T,128] bool mask of real weights)."""
    R, K = ranks.shape
    T = -(-K // TILE)
    full = np.zeros((R, T * TILE), np.int64)
    full[:, :K] = ranks
    real = np.zeros((R, T * TILE), bool)
    real[:, :K] = True
    return full.reshape(-1, TILE), real.reshape(-1, TILE)


def np_rice_choose(r: np.ndarray, real: np.ndarray):
    """binade/rice.py:57-73: per tile (k, qmax, bits); ties to the smaller k; a k whose qmax
    exceeds 63 is illegal (cost = int64 max, so k = 0 keeps the seat only if nothing is legal)."""
    big = np.iinfo(np.int64).max
    n = real.sum(axis=1)
    cost, qmaxes = [], []
    for k in range(KMAX + 1):
        q = r >> k
        qm = q.max(axis=1)
        c = k * n + (np.minimum(q + 1, qm[:, None]) * real).sum(axis=1)
        cost.append(np.where(qm <= QMAX, c, big))
        qmaxes.append(qm)
    cost, qmaxes = np.stack(cost), np.stack(qmaxes)
    k = np.argmin(cost, axis=0)  # first minimum = smallest k
    pick = np.arange(k.size)
    return k, qmaxes[k, pick], cost[k, pick]


def np_rice_encode_ranks(ranks: np.ndarray):
    """binade/rice.py:76-119: ranks [R,K] -> (meta uint8 [R*T], words uint32, roff uint32 [R]).
    Every bit is written once at its own position: low plane bit b of weight i at i*k+b, then
    plane j < qmax with one bit per weight still alive (q >= j), set iff q > j."""
    R, K = ranks.shape
    T = -(-K // TILE)
    r, real = _tile_view(ranks)
    n = real.sum(axis=1)
    k, qmax, tbits = np_rice_choose(r, real)
    per_row = tbits.reshape(R, T)
    row_words = (per_row.sum(axis=1) + 31) >> 5
    roff = np.cumsum(row_words) - row_words
    tile_start = (32 * roff[:, None] + np.cumsum(per_row, axis=1) - per_row).reshape(-1)
    pos, val = [], []
    w_idx = np.arange(TILE)
    for b in range(KMAX):  # low planes
        sel = real & (k[:, None] > b)
        p = tile_start[:, None] + w_idx[None, :] * k[:, None] + b
        pos.append(p[sel])
        val.append(((r >> b) & 1)[sel])
    q = r >> k[:, None]
    plane_start = tile_start + k * n
    for j in range(int(qmax.max()) if qmax.size else 0):
        alive = real & (q >= j) & (qmax[:, None] > j)
        slot = np.cumsum(alive, axis=1) - 1
        p = plane_start[:, None] + slot
        pos.append(p[alive])
        val.append((q > j)[alive])
        plane_start = plane_start + alive.sum(axis=1)
    nwords = int(row_words.sum())
    pos = np.concatenate(pos) if pos else np.zeros(0, np.int64)
    val = np.concatenate(val).astype(np.uint64) if val else np.zeros(0, np.uint64)
    contrib = (val << (pos & 31).astype(np.uint64)).astype(np.float64)  # distinct bits: exact sums
    words = np.bincount(pos >> 5, weights=contrib, minlength=nwords).astype(np.uint64).astype(np.uint32)
    return (k | (qmax << 2)).astype(np.uint8), words, roff.astype(np.uint32)


def _bits_at(words: np.ndarray, pos: np.ndarray) -> np.ndarray:
    idx = pos >> 5
    ok = (idx >= 0) & (idx < words.size)
    w = np.where(ok, words[np.clip(idx, 0, max(words.size - 1, 0))] if words.size else 0, 0)
    return ((w >> (pos & 31).astype(np.uint32)) & 1).astype(np.int64)


def np_rice_decode_ranks(meta, words, roff, K: int):
    """binade/rice.py:128-173: -> (ranks int32 [R,K], end int64 [R] = bit after the row's last
    tile). Tiles of a row are decoded in sequence; rows in parallel."""
    R = roff.size
    T = -(-K // TILE)
    meta = meta.reshape(R, T).astype(np.int64)
    words = np.ascontiguousarray(words, dtype=np.uint32)
    cur = 32 * roff.astype(np.int64)
    out = np.zeros((R, T * TILE), np.int64)
    w_idx = np.arange(TILE)
    for t in range(T):
        n = min(TILE, K - t * TILE)
        k, qmax = meta[:, t] & 3, meta[:, t] >> 2
        real = np.broadcast_to(w_idx < n, (R, TILE))
        low = np.zeros((R, TILE), np.int64)
        for b in range(KMAX):
            sel = real & (k[:, None] > b)
            p = cur[:, None] + w_idx[None, :] * k[:, None] + b
            low |= np.where(sel, _bits_at(words, p), 0) << b
        cur = cur + k * n
        q = np.zeros((R, TILE), np.int64)
        alive = real.copy()
        for j in range(int(qmax.max()) if R else 0):
            alive = alive & (qmax[:, None] > j)
            slot = np.cumsum(alive, axis=1) - 1
            bit = np.where(alive, _bits_at(words, cur[:, None] + slot), 0)
            q += bit
            cur = cur + alive.sum(axis=1)
            alive = alive & (bit == 1)
        out[:, t * TILE : (t + 1) * TILE] = (q << k[:, None]) | low
    return out[:, :K].astype(np.int32), cur


def np_rice_decode(table, meta, words, roff, R: int, K: int) -> np.ndarray:
    """binade/rice.py:176-182: exponents [R,K]; ValueError unless every row ends where the next
    one starts."""
    ranks, end = np_rice_decode_ranks(meta, words, roff, K)
    nxt = np.append(roff[1:].astype(np.int64), words.size)
    if np.any((end + 31) >> 5 != nxt):
        raise ValueError("bit stream length does not match meta")
    return table[ranks]


# ---------------------------------------------------------------------------------------------
# Format 1: fixed-width codes with escapes (binade/format.py)
# ---------------------------------------------------------------------------------------------
F1_ESCAPE = 0x10


def np_f1_choose(r: np.ndarray):
    """binade/format.py:46-60: per tile (b, escape mode) minimising index + escape bits; ties go
    to fixed width, then to the smaller escape width. r: [tiles, 128] ranks."""
    T = r.shape[1]
    rmax = r.max(axis=1).astype(np.int64)
    fixed_b = np.array([int(v).bit_length() for v in rmax], np.int64)
    costs = [T * fixed_b]
    for b in (1, 2, 3, 4):
        costs.append(T * b + 8 * (r >= (1 << b) - 1).sum(axis=1).astype(np.int64))
    pick = np.argmin(np.stack(costs), axis=0)
    return np.where(pick == 0, fixed_b, pick).astype(np.int64), pick > 0


def np_f1_encode(exps: np.ndarray, table: np.ndarray, rank: np.ndarray):
    """binade/format.py:88-101: exponents [R,K] -> (meta uint8 [tiles], idx uint32 words, esc
    uint8). Rows are padded to whole tiles with the most common exponent (rank 0); code i of a
    tile of width b sits at bits i*b .. of the tile's 4*b words, LSB first; in escape mode the
    code 2^b - 1 marks a weight whose exponent byte goes to esc."""
    R, K = exps.shape
    T = -(-K // TILE)
    e = np.full((R, T * TILE), table[0], np.uint8)
    e[:, :K] = exps
    e = e.reshape(-1, TILE)
    r = rank[e].astype(np.int64)
    b, esc_mode = np_f1_choose(r)
    cmax = (1 << b) - 1
    escaped = esc_mode[:, None] & (r >= cmax[:, None])
    codes = np.where(escaped, cmax[:, None], r)
    start = 4 * (np.cumsum(b) - b)  # first word of each tile
    words = np.zeros(4 * int(b.sum()), np.uint64)
    w_idx = np.arange(TILE)
    for t in range(codes.shape[0]):
        if b[t] == 0:
            continue
        pos = w_idx * b[t]
        for bit in range(int(b[t])):
            p = pos + bit
            np.bitwise_or.at(words, start[t] + (p >> 5), ((codes[t] >> bit) & 1).astype(np.uint64) << (p & 31).astype(np.uint64))
    meta = (b | np.where(esc_mode, F1_ESCAPE, 0)).astype(np.uint8)
    return meta, words.astype(np.uint32), e[escaped]


def np_f1_decode(meta, idx, esc, table, R: int, K: int) -> np.ndarray:
    """binade/format.py:104-138: -> exponents [R,K]; ValueError unless the streams are used up
    exactly."""
    T = -(-K // TILE)
    meta = np.asarray(meta).astype(np.int64)
    b, esc_mode = meta & 0x0F, (meta & F1_ESCAPE) != 0
    if meta.size != R * T or 32 * np.asarray(idx).size != TILE * int(b.sum()):
        raise ValueError("format-1 index stream does not fit its tiles")
    start = 32 * 4 * (np.cumsum(b) - b)  # first bit of each tile
    w_idx = np.arange(TILE)
    pos = start[:, None] + w_idx[None, :] * b[:, None]
    codes = np.zeros((meta.size, TILE), np.int64)
    words = np.ascontiguousarray(idx, dtype=np.uint32)
    for bit in range(int(b.max()) if b.size else 0):
        sel = b > bit
        codes[sel] |= _bits_at(words, pos[sel] + bit) << bit
    escaped = esc_mode[:, None] & (codes == ((1 << b) - 1)[:, None])
    if int(escaped.sum()) != np.asarray(esc).size:
        raise ValueError("format-1 escape stream does not fit its tiles")
    e = np.asarray(table)[codes]
    e[escaped] = esc
    return e.reshape(R, T * TILE)[:, :K].astype(np.uint8)


def np_r4_transcode(ranks: np.ndarray, table: np.ndarray) -> dict:
    """binade/mlx/r4.py:143-175 (and its numpy twin binade/mlx/kernel.py:574-598): codes uint16
    [R*T*32] with nibble j = min(rank, 15) of weight 4l+j, flags uint8 [R*T], esc = table[rank]
    of every rank >= 15 in row-major order plus one trailing 0, row_esc = escapes before each row."""
    R, K = ranks.shape
    r, _ = _tile_view(ranks)
    q = np.minimum(r, 15).astype(np.uint16).reshape(-1, 32, 4)
    codes = q[..., 0] | (q[..., 1] << 4) | (q[..., 2] << 8) | (q[..., 3] << 12)
    hit = r >= 15
    per_tile = hit.sum(axis=1)
    per_row = per_tile.reshape(R, -1).sum(axis=1)
    return {
        "codes": codes.reshape(-1),
        "flags": (per_tile > 0).astype(np.uint8),
        "esc": np.concatenate([table[r[hit]], np.zeros(1, np.uint8)]).astype(np.uint8),
        "row_esc": (np.cumsum(per_row) - per_row).astype(np.uint32),
    }


def np_r4_ranks(a: dict, R: int, K: int) -> np.ndarray:
    """Exponents [R,K] of an R4 matrix (the decode rule of binade/mlx/cuda_kernels.py:853-892):
    nibble c < 15 -> table[c]; c == 15 -> the next escape byte of the row, in column order."""
    T = -(-K // TILE)
    codes = a["codes"].reshape(R, T * 32).astype(np.uint16)
    nib = np.stack([(codes >> s) & 15 for s in (0, 4, 8, 12)], axis=-1).reshape(R, T * TILE)[:, :K]
    e = a["table"][nib]
    hit = nib == 15
    pos = a["row_esc"].astype(np.int64)[:, None] + np.cumsum(hit, axis=1) - 1
    return np.where(hit, a["esc"][np.clip(pos, 0, a["esc"].size - 1)], e).astype(np.uint8)


def np_r4_dense(a: dict, R: int, K: int) -> np.ndarray:
    return np_join(a["raw"].reshape(R, K), np_r4_ranks(a, R, K))


def bf16_to_f32(u: np.ndarray) -> np.ndarray:
    return (u.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(f: np.ndarray) -> np.ndarray:
    """Round to nearest even; NaN -> 0x7FFF (what the GPU's cvt.rn.bf16.f32 gives)."""
    v = np.ascontiguousarray(f, np.float32).view(np.uint32).astype(np.uint64)
    out = ((v + 0x7FFF + ((v >> 16) & 1)) >> 16).astype(np.uint16)
    return np.where(np.isnan(f), np.uint16(0x7FFF), out)


def np_rows_same_order(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    """Y [M,N] BF16 words = X [M,K] . W[N,K]^T in the documented summation order: lane l owns
    weights 128t+4l+j, accumulates in fp32 over t then j (absent columns skipped), lanes combine
    with strides 16, 8, 4, 2, 1, one rounding to BF16. Products of two BF16 values are exact in
    fp32 in the normal range, so multiply-then-add equals the kernel's fused multiply-add there
    (restates the order of binade/mlx/cuda_kernels.py:70-92, n = 4)."""
    M, K = x.shape
    N = w.shape[0]
    T = -(-K // TILE)
    xf = np.zeros((M, T * TILE), np.float32)
    xf[:, :K] = bf16_to_f32(x)
    wf = np.zeros((N, T * TILE), np.float32)
    wf[:, :K] = bf16_to_f32(w)
    real = (np.arange(T * TILE) < K).reshape(T, 32, 4)
    xf, wf = xf.reshape(M, 1, T, 32, 4), wf.reshape(1, N, T, 32, 4)
    acc = np.zeros((M, N, 32), np.float32)
    for t in range(T):
        for j in range(4):
            step = acc + wf[:, :, t, :, j] * xf[:, :, t, :, j]
            acc = np.where(real[t, :, j][None, None, :], step, acc).astype(np.float32)
    for s in (16, 8, 4, 2, 1):
        acc = (acc[..., :s] + acc[..., s : 2 * s]).astype(np.float32)
    return f32_to_bf16(acc[..., 0])


# ----------------------------------------------------------------------------- C
_lib = None


def build(force: bool = False) -> Path:
    """Compile binade_oracle.c (gcc, a second or two). Building the checker is not using it."""
    if force or not LIB.exists() or LIB.stat().st_mtime < (HERE / "binade_oracle.c").stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE)] + (["-B"] if force else []), check=True, capture_output=True)
    return LIB


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(str(LIB))
        _lib.bo_rice_encode_ranks.restype = ctypes.c_int64
        _lib.bo_r4_transcode.restype = ctypes.c_int64
    return _lib


def _p(a):
    return None if a is None else ctypes.c_void_p(a.ctypes.data)


def _i(v):
    return ctypes.c_int64(int(v))


def set_threads(n: int) -> int:
    """OpenMP threads of the C oracle's row loops; returns the count in effect."""
    return int(lib().bo_set_threads(ctypes.c_int(n)))


def c_rank_table(hist):
    table, rank = np.zeros(256, np.uint8), np.zeros(256, np.uint8)
    lib().bo_rank_table(_p(np.ascontiguousarray(hist, np.int64)), _p(table), _p(rank))
    return table, rank


def c_rice_encode_ranks(ranks):
    ranks = np.ascontiguousarray(ranks, np.uint8)
    R, K = ranks.shape
    T = -(-K // TILE)
    meta, roff = np.zeros(R * T, np.uint8), np.zeros(R, np.uint32)
    n = lib().bo_rice_encode_ranks(_p(ranks), _i(R), _i(K), _p(meta), None, _i(0), _p(roff))
    words = np.zeros(n, np.uint32)
    got = lib().bo_rice_encode_ranks(_p(ranks), _i(R), _i(K), _p(meta), _p(words), _i(n), _p(roff))
    assert got == n
    return meta, words, roff


def c_rice_decode_ranks(meta, words, roff, K):
    R = roff.size
    meta, words, roff = (np.ascontiguousarray(a, d) for a, d in ((meta, np.uint8), (words, np.uint32), (roff, np.uint32)))
    ranks, end = np.zeros((R, K), np.uint8), np.zeros(R, np.int64)
    lib().bo_rice_decode_ranks(_p(meta), _p(words), _i(words.size), _p(roff), _i(R), _i(K), _p(ranks), _p(end))
    return ranks, end


def c_r4_transcode(ranks, table) -> dict:
    ranks = np.ascontiguousarray(ranks, np.uint8)
    table = np.ascontiguousarray(table, np.uint8)
    R, K = ranks.shape
    T = -(-K // TILE)
    codes, flags, row_esc = np.zeros(R * T * 32, np.uint16), np.zeros(R * T, np.uint8), np.zeros(R, np.uint32)
    n = lib().bo_r4_transcode(_p(ranks), _p(table), _i(R), _i(K), None, None, None, None)
    esc = np.zeros(n + 1, np.uint8)
    lib().bo_r4_transcode(_p(ranks), _p(table), _i(R), _i(K), _p(codes), _p(flags), _p(esc), _p(row_esc))
    return {"codes": codes, "flags": flags, "esc": esc, "row_esc": row_esc}


def _r4_args(a):
    return [np.ascontiguousarray(a[k], d) for k, d in (("raw", np.uint8), ("codes", np.uint16), ("flags", np.uint8), ("esc", np.uint8), ("table", np.uint8), ("row_esc", np.uint32))]


def c_r4_dense(a: dict, N: int, K: int, nb=None, rs=None, r0: int = 0) -> np.ndarray:
    raw, codes, flags, esc, table, row_esc = _r4_args(a)
    out = np.zeros((N, K), np.uint16)
    nb = nb or N
    lib().bo_r4_dense(_p(raw), _p(codes), _p(flags), _p(esc), _p(table), _p(row_esc), _i(N), _i(K), _i(nb), _i(rs or nb), _i(r0), _p(out))
    return out


def c_r4_gather(a: dict, x, xi, ei, n: int, K: int, rs: int, r0: int = 0) -> np.ndarray:
    raw, codes, _, esc, table, row_esc = _r4_args(a)
    x = np.ascontiguousarray(x, np.uint16)
    xi, ei = np.ascontiguousarray(xi, np.uint32), np.ascontiguousarray(ei, np.uint32)
    y = np.zeros((ei.size, n), np.uint16)
    lib().bo_r4_gather(_p(x), _p(raw), _p(codes), _p(esc), _p(table), _p(row_esc), _p(xi), _p(ei), _i(ei.size), _i(n), _i(K), _i(rs), _i(r0), _p(y))
    return y


def c_r4_matvec(a: dict, x, N: int, K: int) -> np.ndarray:
    z = np.zeros(1, np.uint32)
    return c_r4_gather(a, x, z, z, N, K, 0, 0)[0]


def c_dense_rows(x, w) -> np.ndarray:
    x, w = np.ascontiguousarray(x, np.uint16), np.ascontiguousarray(w, np.uint16)
    y = np.zeros((x.shape[0], w.shape[0]), np.uint16)
    lib().bo_dense_rows(_p(x), _p(w), _i(x.shape[0]), _i(w.shape[0]), _i(x.shape[1]), _p(y))
    return y


def c_ranks_of(w):
    w = np.ascontiguousarray(w, np.uint16)
    raw, ranks, table = np.zeros(w.shape, np.uint8), np.zeros(w.shape, np.uint8), np.zeros(256, np.uint8)
    lib().bo_ranks_of(_p(w), _i(w.size), _p(raw), _p(table), _p(ranks))
    return raw, table, ranks


def esc_columns(a: dict):
    """The derived arrays of bn_r4_esc_columns for an R4 dict of this module: (esc_cols uint8
    [n_esc + 8], col_esc uint16 [R, 16]). Every row's run of escape bytes is regrouped by column
    c = (k % 128) // 8 of the escaped weight k (row order kept inside a column); col_esc[r, c]
    counts the row's escapes in columns below c. Not a reference structure: it restates the
    definition in include/binade_b200.h so that the GPU builder can be checked."""
    K = a["shape"][-1]
    R = a["row_esc"].size
    T = -(-K // TILE)
    codes = np.ascontiguousarray(a["codes"], np.uint16).reshape(R, T * 32)
    nib = np.stack([(codes >> (4 * j)) & 15 for j in range(4)], axis=-1).reshape(R, T * TILE)
    rows, ks = np.nonzero(nib == 15)  # row-major: the order of `esc`
    col = (ks % TILE) // 8
    n = rows.size
    esc = np.ascontiguousarray(a["esc"], np.uint8)
    if n != esc.size - 1:
        raise ValueError(f"{n} codes 15 but {esc.size - 1} escape bytes")
    order = np.lexsort((np.arange(n), col, rows))
    esc_cols = np.zeros(n + 8, np.uint8)
    esc_cols[:n] = esc[:n][order]
    per = np.zeros((R, 16), np.int64)
    np.add.at(per, (rows, col), 1)
    col_esc = (np.cumsum(per, axis=1) - per).astype(np.uint16)
    return esc_cols, col_esc


def pack_r4(w: np.ndarray) -> dict:
    """BF16 words [R,K] -> full R4 dict via the C oracle (for building kernel test inputs)."""
    R, K = w.shape
    raw, table, ranks = c_ranks_of(w)
    a = c_r4_transcode(ranks, table)
    a.update(raw=raw, table=table, shape=(R, K))
    return a
