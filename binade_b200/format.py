"""Constants and the per-tensor rank table shared by both on-disk formats.

A tensor's 256-entry table lists its exponent bytes by descending frequency; every weight
stores the rank of its exponent (reference: binade/format.py:17,34-42). Format 1 (fixed-width
codes with escapes) is read on the GPU (`cuda.kernels.Format1`) but not written; format 2 lives
in `rice`.
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
