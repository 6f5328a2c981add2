"""Constants and the per-tensor rank table shared by both on-disk formats.

A tensor's 256-entry table lists its exponent bytes by descending frequency; every weight
stores the rank of its exponent (reference: binade/format.py:17,34-42). Format 1 (fixed-width
codes with escapes) is written here on host cores (`encode_words`) and read on the GPU
(`cuda.kernels.Format1`); format 2 lives in `rice`.
"""

from __future__ import annotations

import numpy as np

from . import _native

TILE = 128  # weights per tile, along K, never crossing a row


def rank_table(hist: np.ndarray):
    """(table [256] uint8: exponent of each rank, rank [256] uint8: rank of each exponent).

    Exponents sort by descending count; equal counts keep ascending exponent order; table
    entries of exponents that never occur are 0."""
    hist = np.ascontiguousarray(hist, np.int64)
    if hist.shape != (256,):
        raise ValueError(f"expected a 256-bin histogram, got shape {hist.shape}")
    table, rank = np.empty(256, np.uint8), np.empty(256, np.uint8)
    _native.call("host", "bn_host_rank_table", _native.nptr(hist), _native.nptr(table), _native.nptr(rank))
    return table, rank


def encode_words(w: np.ndarray, rank: np.ndarray, threads: int = 0):
    """Format 1 (reference: binade/format.py:46-101) straight from BF16 words [R, K] with the
    tensor's rank table -> (meta uint8 [R * ceil(K/128)], idx uint32 words, esc uint8). Per tile
    the cheapest of a fixed width (the largest rank's bit length) and escape widths 1..4; a tile
    of width b is 4 b words, code i at bits i b .., LSB first; escaped weights put their exponent
    byte into esc, in tensor order. Rows are padded to whole tiles with rank 0."""
    w = np.ascontiguousarray(w, np.uint16)
    rank = np.ascontiguousarray(rank, np.uint8)
    if w.ndim != 2:
        raise ValueError("words must be [R, K]")
    R, K = w.shape
    T = -(-K // TILE) if K else 0
    if R == 0 or K == 0:
        return np.zeros(R * T, np.uint8), np.zeros(0, np.uint32), np.zeros(0, np.uint8)
    meta = np.empty(R * T, np.uint8)
    counts = np.zeros(2, np.uint64)
    lead = (_native.nptr(w), _native.nptr(rank), R, K, _native.nptr(meta))
    _native.call("host", "bn_host_f1_encode", *lead, None, 0, None, 0, _native.nptr(counts), threads, ok=(_native.ERR_CAPACITY,))
    idx, esc = np.empty(int(counts[0]), np.uint32), np.empty(int(counts[1]), np.uint8)
    _native.call("host", "bn_host_f1_encode", *lead, _native.nptr(idx), idx.size, _native.nptr(esc), esc.size, _native.nptr(counts), threads)
    return meta, idx, esc
