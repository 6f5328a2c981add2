"""Python face of the CUDA entry points (include/binade_b200.h) on torch CUDA tensors.

Mirrors the reference's kernel wrappers (binade/mlx/cuda_kernels.py: rice_ranks, r4_matvec,
r4_gather, r4_decode) with torch tensors in place of MLX arrays. Tensors are only carriers of
device memory: every call passes raw pointers and the current CUDA stream to the C ABI.
Nothing here runs without a CUDA device and the built library.
"""

from __future__ import annotations

import ctypes

import numpy as np
import torch

from .. import _native
from ..format import TILE

R4_KEYS = ("raw", "codes", "flags", "esc", "table", "row_esc")
NO_EXPERT = -1  # BN_NO_EXPERT (0xFFFFFFFF) in an int32 tensor: the expert id of a padding slot


def require_cuda() -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("binade_b200 needs a CUDA device: its kernels have no CPU fallback")
    return torch.device("cuda", torch.cuda.current_device())


def to_device(a, dtype=None) -> torch.Tensor:
    """numpy array or tensor -> contiguous CUDA tensor (uint16/uint32 travel as int16/int32)."""
    dev = require_cuda()
    if isinstance(a, np.ndarray):
        if a.dtype == np.uint16:
            a = a.view(np.int16)
        elif a.dtype == np.uint32:
            a = a.view(np.int32)
        a = torch.from_numpy(np.ascontiguousarray(a))
    t = a.to(dev, non_blocking=True).contiguous()
    return t if dtype is None else t.to(dtype)


def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    """The current CUDA stream's handle (the raw query: building a torch Stream object per kernel
    call costs more host time than the launch)."""
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


def _call(fn, *args):
    return _native.call("cuda", fn, *args, _stream())


def r4_struct(a: dict) -> _native.R4Struct:
    """bn_r4 of an R4 dict; the column-ordered escapes ride along when the dict holds them."""
    cols = (a["esc_cols"].data_ptr(), a["col_esc"].data_ptr()) if "esc_cols" in a else (None, None)
    return _native.R4Struct(*(a[k].data_ptr() for k in R4_KEYS), a["esc"].numel() - 1, *cols)


def r4_esc_columns(a: dict) -> None:
    """Adds `esc_cols` (uint8 [n_esc + 8]) and `col_esc` (int16-typed uint16 [rows, 16]) to an R4
    dict: every row's escape bytes regrouped by column of eight weights, which lets a thread of
    the batch-1 kernels walk its own escapes (bn_r4_esc_columns). Shapes the kernels do not take
    (K % 16) are left alone."""
    rows, K = a["raw"].shape
    if "esc_cols" in a or K % 16 or K > 65520:
        return
    dev = a["raw"].device
    esc_cols = torch.empty(a["esc"].numel() - 1 + 8, dtype=torch.uint8, device=dev)
    col_esc = torch.empty((rows, 16), dtype=torch.int16, device=dev)
    _call("bn_r4_esc_columns", ctypes.byref(r4_struct(a)), rows, K, _p(esc_cols), _p(col_esc))
    a["esc_cols"], a["col_esc"] = esc_cols, col_esc


def split_hist(u: torch.Tensor):
    """int16 BF16 words (any shape, contiguous, on the device) -> (raw uint8 [numel], hist int64
    numpy [256] of the exponent bytes; reading the histogram synchronises)."""
    raw = torch.empty(u.numel(), dtype=torch.uint8, device=u.device)
    hist = torch.empty(256, dtype=torch.int32, device=u.device)
    _call("bn_bf16_split_hist", _p(u), u.numel(), _p(raw), _p(hist))
    return raw, hist.cpu().numpy().view(np.uint32).astype(np.int64)


def rice_encode_ranked(u: torch.Tensor, rank_d: torch.Tensor):
    """int16 BF16 words [R, K] on the device and the device copy of the exponent -> rank table ->
    (meta uint8 [R*T], bits int32 [nwords], roff int32 [R]) of these rows' own stream."""
    R, K = u.shape
    T = -(-K // TILE)
    dev = u.device
    meta = torch.empty(R * T, dtype=torch.uint8, device=dev)
    row_words, roff = torch.empty(R, dtype=torch.int32, device=dev), torch.empty(R, dtype=torch.int32, device=dev)
    total = torch.zeros(1, dtype=torch.int64, device=dev)
    _call("bn_rice_encode_plan", _p(u), _p(rank_d), R, K, _p(meta), _p(row_words), _p(roff), _p(total))
    nwords = int(total.item())
    if nwords >= 1 << 32:
        raise ValueError(f"{nwords} words overflow uint32 row offsets")
    bits = torch.empty(nwords, dtype=torch.int32, device=dev)
    _call("bn_rice_encode_write", _p(u), _p(rank_d), _p(meta), _p(roff), R, K, _p(bits) if nwords else None, nwords)
    return meta, bits, roff


def rice_encode(w: torch.Tensor) -> dict:
    """BF16 weights [.., K] on the device (bfloat16 or int16 words) -> the format-2 arrays as
    device tensors {"raw", "table", "meta", "bits", "roff", "shape"}, bit for bit what the host
    packer writes (pack.pack). Two small host reads on the way: the exponent histogram (the rank
    table is built on the host like the reference does) and the stream's length in words."""
    from ..format import rank_table

    shape = tuple(w.shape)
    u = w.contiguous().view(torch.int16).reshape(-1, shape[-1])
    raw, hist = split_hist(u)
    table, rank = rank_table(hist)
    meta, bits, roff = rice_encode_ranked(u, to_device(rank))
    return {"raw": raw.reshape(shape), "table": to_device(table), "meta": meta, "bits": bits, "roff": roff, "shape": shape}


def rice_ranks(meta: torch.Tensor, bits: torch.Tensor, roff: torch.Tensor, K: int):
    """(ranks uint8 [R, ceil(K/128)*128], rend int32-typed uint32 [R])."""
    R, T = roff.numel(), -(-K // TILE)
    if meta.numel() != R * T:
        raise ValueError(f"{meta.numel()} tiles for {R} rows of {K}")
    ranks = torch.empty((R, T * TILE), dtype=torch.uint8, device=meta.device)
    rend = torch.empty(R, dtype=torch.int32, device=meta.device)
    if bits.numel() == 0:
        bits = torch.zeros(1, dtype=torch.int32, device=meta.device)
        nwords = 0
    else:
        nwords = bits.numel()
    _call("bn_rice_ranks", _p(meta), _p(bits), nwords, _p(roff), R, K, _p(ranks), _p(rend))
    return ranks, rend


def rice_unpack(meta, bits, roff, table, raw, R: int, K: int):
    """BF16 rows [R, K] (bfloat16 tensor) and rend [R] from a Rice stream plus raw bytes."""
    out = torch.empty((R, K), dtype=torch.bfloat16, device=raw.device)
    rend = torch.empty(R, dtype=torch.int32, device=raw.device)
    nwords = bits.numel()
    if nwords == 0:
        bits = torch.zeros(1, dtype=torch.int32, device=raw.device)
    _call("bn_rice_unpack", _p(meta), _p(bits), nwords, _p(roff), _p(table), _p(raw), R, K, _p(out), _p(rend))
    return out, rend


def rice_to_r4(meta, bits, roff, table, R: int, K: int, esc_cap: int | None = None):
    """The load-time expander: Rice arrays on the device -> (codes, flags, esc, row_esc, bad_row).

    One host read of 32 bytes of counters per tensor (escape total, scratch claimed, first bad
    row); the scratch is sized from the tile count and grown once if a tensor needs more."""
    dev = meta.device
    T = -(-K // TILE)
    codes = torch.empty(R * T * 32, dtype=torch.int16, device=dev)
    flags = torch.empty(R * T, dtype=torch.uint8, device=dev)
    row_cnt = torch.empty(R, dtype=torch.int32, device=dev)
    tmp_off = torch.empty(R, dtype=torch.int32, device=dev)
    counters = torch.empty(8, dtype=torch.int32, device=dev)
    nwords = bits.numel()
    if nwords == 0:
        bits = torch.zeros(1, dtype=torch.int32, device=dev)
    cap = esc_cap if esc_cap is not None else 4096 + R * K // 4  # rows claim an upper bound, about 1/7 of the weights on real data
    while True:
        cap = min(cap, (1 << 32) - 1)
        esc_tmp = torch.empty(cap, dtype=torch.uint8, device=dev)
        _call("bn_rice_to_r4", _p(meta), _p(bits), nwords, _p(roff), _p(table), R, K, _p(codes), _p(flags), _p(row_cnt), _p(esc_tmp), cap, _p(tmp_off), _p(counters))
        c = counters.cpu().numpy().view(np.uint32)
        claimed = int(c[4]) | int(c[5]) << 32
        if claimed <= cap:
            break
        if claimed >= 1 << 32:
            raise ValueError("escape scratch of one call exceeds 4 GiB: expand the tensor in row chunks")
        cap = claimed
    n_esc = int(c[2])
    bad_row = R - int(c[1]) if c[1] else -1
    esc = torch.empty(n_esc + 1, dtype=torch.uint8, device=dev)
    _call("bn_r4_finish", _p(row_cnt), _p(esc_tmp), _p(tmp_off), R, _p(row_cnt), _p(esc), n_esc + 1)
    return codes, flags, esc, row_cnt, bad_row


class Format1:
    """Format-1 file arrays of one tensor on the device plus the row offsets the format does not
    store (rebuilt by bn_f1_offsets). Raises ValueError when meta and idx disagree with the array
    sizes, as format.decode does (binade/format.py:128-133)."""

    def __init__(self, meta, idx, esc, table, R: int, K: int):
        self.R, self.K = R, K
        T = -(-K // TILE)
        self.meta, self.table = to_device(meta).reshape(-1), to_device(table)
        dev = self.meta.device
        if self.meta.numel() != R * T:
            raise ValueError(f"{self.meta.numel()} tiles for {R} rows of {K}")
        idx, esc = to_device(idx).reshape(-1), to_device(esc).reshape(-1)
        self.nwords, self.n_esc = idx.numel(), esc.numel()
        self.idx = idx if self.nwords else torch.zeros(1, dtype=torch.int32, device=dev)
        self.esc = esc if self.n_esc else torch.zeros(1, dtype=torch.uint8, device=dev)
        self.woff = torch.empty(max(R, 1), dtype=torch.int32, device=dev)
        self.eoff = torch.empty(max(R, 1), dtype=torch.int32, device=dev)
        if R:
            scratch = torch.empty(2 * R, dtype=torch.int32, device=dev)
            totals = torch.zeros(2, dtype=torch.int32, device=dev)
            _call("bn_f1_offsets", _p(self.meta), _p(self.idx), self.nwords, R, K, _p(self.woff), _p(self.eoff), _p(scratch), _p(totals))
            words, escapes = (int(v) for v in totals.cpu().numpy().view(np.uint32))
            if words != self.nwords or escapes != self.n_esc:
                raise ValueError(f"format-1 streams do not fit their tiles: {words} index words and {escapes} escapes expected, {self.nwords} and {self.n_esc} given")

    @staticmethod
    def rows_of(whole: "Format1", r0: int, r1: int) -> "Format1":
        """Rows r0 .. r1 - 1 of an already indexed tensor, sharing its arrays: the row offsets are
        absolute, so a row range is a view of meta, woff and eoff."""
        T = -(-whole.K // TILE)
        part = object.__new__(Format1)
        part.R, part.K = r1 - r0, whole.K
        part.meta, part.table = whole.meta[r0 * T : r1 * T], whole.table
        part.idx, part.esc, part.nwords, part.n_esc = whole.idx, whole.esc, whole.nwords, whole.n_esc
        part.woff, part.eoff = whole.woff[r0:r1], whole.eoff[r0:r1]
        return part

    def _head(self):
        return (_p(self.meta), _p(self.idx), self.nwords, _p(self.woff), _p(self.esc), self.n_esc, _p(self.eoff), _p(self.table))

    def ranks(self) -> torch.Tensor:
        """8-bit ranks [R, T*128] (padding columns 0)."""
        T = -(-self.K // TILE)
        out = torch.empty((self.R, T * TILE), dtype=torch.uint8, device=self.meta.device)
        if self.R:
            _call("bn_f1_ranks", *self._head(), self.R, self.K, _p(out))
        return out

    def unpack(self, raw) -> torch.Tensor:
        """BF16 rows [R, K] from the raw sign+mantissa bytes."""
        out = torch.empty((self.R, self.K), dtype=torch.bfloat16, device=self.meta.device)
        if self.R:
            _call("bn_f1_unpack", *self._head(), _p(to_device(raw)), self.R, self.K, _p(out))
        return out

    def to_r4(self, esc_cap: int | None = None):
        """(codes, flags, esc, row_esc) of the R4 layout: the expander for format-1 files."""
        dev, R, K = self.meta.device, self.R, self.K
        T = -(-K // TILE)
        codes = torch.empty(R * T * 32, dtype=torch.int16, device=dev)
        flags = torch.empty(R * T, dtype=torch.uint8, device=dev)
        row_cnt = torch.empty(R, dtype=torch.int32, device=dev)
        tmp_off = torch.empty(R, dtype=torch.int32, device=dev)
        counters = torch.empty(8, dtype=torch.int32, device=dev)
        cap = esc_cap if esc_cap is not None else 4096 + R * K // 4
        while True:
            cap = min(cap, (1 << 32) - 1)
            esc_tmp = torch.empty(cap, dtype=torch.uint8, device=dev)
            _call("bn_f1_to_r4", *self._head(), R, K, _p(codes), _p(flags), _p(row_cnt), _p(esc_tmp), cap, _p(tmp_off), _p(counters))
            c = counters.cpu().numpy().view(np.uint32)
            claimed = int(c[4]) | int(c[5]) << 32
            if claimed <= cap:
                break
            if claimed >= 1 << 32:
                raise ValueError("escape scratch of one call exceeds 4 GiB: expand the tensor in row chunks")
            cap = claimed
        n_esc = int(c[2])
        esc = torch.empty(n_esc + 1, dtype=torch.uint8, device=dev)
        _call("bn_r4_finish", _p(row_cnt), _p(esc_tmp), _p(tmp_off), R, _p(row_cnt), _p(esc), n_esc + 1)
        return codes, flags, esc, row_cnt


def r4_decode(a: dict, N: int, K: int, nb: int | None = None, rs: int | None = None, r0: int = 0) -> torch.Tensor:
    """BF16 [N, K] from R4; output row r is storage row (r // nb) * rs + r0 + r % nb."""
    out = torch.empty((N, K), dtype=torch.bfloat16, device=a["raw"].device)
    nb = nb or max(N, 1)
    _call("bn_r4_decode", ctypes.byref(r4_struct(a)), N, K, nb, rs or nb, r0, _p(out))
    return out


def r4_gather_grouped(a: dict, x: torch.Tensor, xi: torch.Tensor, ei: torch.Tensor, E: int, max_per_expert: int, n: int, rs: int, r0: int, K: int, split: int | None = None):
    """r4_gather's outputs with every expert's rows read once for all its slots: the slots are
    sorted by expert on the device (no host sync) and each expert multiplies up to 8 input rows
    per pass. ei: int32 [G] expert of each slot (0 <= ei < E); max_per_expert bounds the slots of
    one expert (the token count when a token names an expert at most once). K % 16 == 0.
    Slots whose expert id is NO_EXPERT (padding) sort behind every expert and are skipped."""
    G = ei.numel()
    dev = x.device
    bucket = torch.clamp(ei.to(torch.int64) & 0xFFFFFFFF, max=E)  # padding slots: one bucket past the experts
    order = torch.argsort(bucket, stable=True).to(torch.int32)
    counts = torch.zeros(E + 1, dtype=torch.int32, device=dev).scatter_add_(0, bucket, torch.ones(G, dtype=torch.int32, device=dev))  # (bincount would synchronise)
    seg = torch.zeros(E + 1, dtype=torch.int32, device=dev)
    seg[1:] = torch.cumsum(counts[:E], 0).to(torch.int32)
    if split:
        y = torch.empty((G, split), dtype=torch.bfloat16, device=dev)
        y2 = torch.empty((G, n - split), dtype=torch.bfloat16, device=dev)
    else:
        y, y2 = torch.empty((G, n), dtype=torch.bfloat16, device=dev), None
    _call("bn_r4_gather_grouped", _p(x), ctypes.byref(r4_struct(a)), _p(xi), _p(seg), _p(order), E, G, max_per_expert, n, K, rs, r0, split or 0, _p(y), _p(y2))
    return (y, y2) if split else y


def r4_mma(a: dict, x: torch.Tensor, N: int, K: int, split: int = 1) -> torch.Tensor:
    """x [M, K] (1 <= M <= 256, bfloat16, contiguous rows, K % 8 == 0) -> [M, N] through the fused
    decode GEMM on the tensor cores (tcgen05); accumulation order is the hardware's. split: the K
    tiles in that many equal slices, summed apart and added in fp32 (cuBLAS's split-K order)."""
    M = x.shape[0]
    y = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    _call("bn_r4_mma_split", _p(x), x.stride(0), ctypes.byref(r4_struct(a)), M, N, K, _p(y), N, split)
    return y


def r4_lookup(a: dict, ids: torch.Tensor, N: int, K: int) -> torch.Tensor:
    """BF16 rows [n, K] of an R4 table of N rows for ids [n] (int32 on the device); an id outside
    the table gives a row of zeros."""
    out = torch.empty((ids.numel(), K), dtype=torch.bfloat16, device=a["raw"].device)
    if ids.numel() == 0:
        return out
    _call("bn_r4_lookup", ctypes.byref(r4_struct(a)), N, _p(ids), ids.numel(), K, _p(out))
    return out


def rice_lookup(meta, bits, roff, table, raw, N: int, K: int, ids: torch.Tensor) -> torch.Tensor:
    """BF16 rows [n, K] for ids [n] (int32 on the device) of an N x K table kept as a Rice stream;
    an id outside the table gives a row of zeros."""
    out = torch.empty((ids.numel(), K), dtype=torch.bfloat16, device=raw.device)
    if ids.numel() == 0:
        return out
    nwords = bits.numel()
    if nwords == 0:
        bits = torch.zeros(1, dtype=torch.int32, device=raw.device)
    _call("bn_rice_lookup", _p(meta), _p(bits), nwords, _p(roff), _p(table), _p(raw), N, K, _p(ids), ids.numel(), _p(out))
    return out


def r4_rows(a: dict, x: torch.Tensor, N: int, K: int) -> torch.Tensor:
    """x [M, K] (1 <= M <= 16, bfloat16, contiguous rows) -> [M, N], fused decode."""
    M = x.shape[0]
    y = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    _call("bn_r4_rows", _p(x), x.stride(0), ctypes.byref(r4_struct(a)), M, N, K, _p(y), N)
    return y


def r4_matvec(a: dict, x: torch.Tensor, N: int, K: int, struct=None) -> torch.Tensor:
    """x [..., K] holding one row -> [..., N] (reference: r4_matvec, cuda_kernels.py:118-130).
    `struct`: the bn_r4 of `a` when the caller keeps one (saves rebuilding it per call)."""
    y = torch.empty((*x.shape[:-1], N), dtype=torch.bfloat16, device=x.device)
    _call("bn_r4_rows", _p(x), K, ctypes.byref(struct if struct is not None else r4_struct(a)), 1, N, K, _p(y), N)
    return y


class R4Group:
    """Up to four R4 matrices of the same K whose batch-1 products share their input: one launch
    for all of them (bn_r4_rows_multi). Keeps the bn_r4 structs and the pointer arrays alive."""

    def __init__(self, structs, Ns, K: int):
        if not 1 <= len(structs) <= 4:
            raise ValueError("a group holds one to four matrices")
        self.structs, self.Ns, self.K = list(structs), [int(n) for n in Ns], int(K)
        n = len(self.structs)
        self._w = (ctypes.c_void_p * n)(*[ctypes.addressof(s) for s in self.structs])
        self._n = (ctypes.c_int64 * n)(*self.Ns)

    def __call__(self, x: torch.Tensor):
        """x [..., K] holding one row -> list of [..., N_i]."""
        ys = [torch.empty((*x.shape[:-1], n), dtype=torch.bfloat16, device=x.device) for n in self.Ns]
        yp = (ctypes.c_void_p * len(ys))(*[y.data_ptr() for y in ys])
        _call("bn_r4_rows_multi", _p(x), ctypes.cast(self._w, ctypes.c_void_p), ctypes.cast(self._n, ctypes.c_void_p), len(ys), self.K, ctypes.cast(yp, ctypes.c_void_p))
        return ys


def r4_gather(a: dict, x: torch.Tensor, xi: torch.Tensor, ei: torch.Tensor, n: int, rs: int, r0: int, K: int, split: int | None = None, shape: tuple | None = None):
    """[G, n] (or `shape`), or with split the pair [G, split], [G, n - split]
    (reference: r4_gather, cuda_kernels.py:133-146). xi, ei: int32 tensors of G entries."""
    G = ei.numel()
    dev = x.device
    if split:
        y = torch.empty((G, split), dtype=torch.bfloat16, device=dev)
        y2 = torch.empty((G, n - split), dtype=torch.bfloat16, device=dev)
    else:
        y, y2 = torch.empty(shape or (G, n), dtype=torch.bfloat16, device=dev), None
    _call("bn_r4_gather", _p(x), ctypes.byref(r4_struct(a)), _p(xi), _p(ei), G, n, K, rs, r0, split or 0, _p(y), _p(y2))
    return (y, y2) if split else y
