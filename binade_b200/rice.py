"""Format 2: Rice codes over per-tensor frequency ranks (reference: binade/rice.py).

Tile = 128 weights of one row (the last tile of a row may be shorter). Per tile the encoder
picks k in 0..3 minimising the tile's bits, q = rank >> k:
  meta  k | qmax << 2
  bits  low plane (bit b of weight i at i*k + b), then planes j = 0 .. qmax-1 with one bit per
        weight whose q >= j, set iff q > j; LSB first in little-endian uint32 words
  roff  first word of each row (rows start on a word boundary)

Encoding runs on the host in C++ (all cores); decoding runs on the GPU. There is no numpy
decoder in this package: `decode*` need a CUDA device.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np

from . import _native
from .format import TILE

KMAX = 3
QMAX = 63


@dataclass
class RiceEncoded:
    table: np.ndarray  # uint8 [256]
    meta: np.ndarray  # uint8 [ntiles]
    bits: np.ndarray  # uint32 [words]
    roff: np.ndarray  # uint32 [rows]

    def nbits(self) -> int:
        """Exponent-side payload in bits (the raw sign+mantissa bytes are not counted)."""
        return 8 * self.table.size + 8 * self.meta.size + 32 * self.bits.size + 32 * self.roff.size


def tiles_per_row(K: int, T: int = TILE) -> int:
    return -(-K // T)


def _encode(fn: str, lead: tuple, R: int, K: int, threads: int):
    meta = np.empty(R * tiles_per_row(K), np.uint8)
    roff = np.empty(R, np.uint32)
    n = ctypes.c_uint64(0)
    _native.call("host", fn, *lead, R, K, _native.nptr(meta), _native.nptr(roff), None, 0, ctypes.byref(n), threads, ok=(_native.ERR_CAPACITY,))
    if n.value >= 1 << 32:
        raise ValueError(f"{n.value} words overflow uint32 row offsets")
    words = np.empty(n.value, np.uint32)
    _native.call("host", fn, *lead, R, K, _native.nptr(meta), _native.nptr(roff), _native.nptr(words), n.value, ctypes.byref(n), threads)
    return meta, words, roff


def encode_ranks(ranks: np.ndarray, threads: int = 0):
    """[R, K] ranks (0..255) -> (meta uint8 [R * ceil(K/128)], words uint32, roff uint32 [R])."""
    ranks = np.ascontiguousarray(ranks)
    if ranks.ndim != 2:
        raise ValueError("ranks must be [R, K]")
    if ranks.dtype != np.uint8:
        if ranks.size and (ranks.min() < 0 or ranks.max() > 255):
            raise ValueError("ranks must fit 8 bits")
        ranks = ranks.astype(np.uint8)
    R, K = ranks.shape
    if R == 0 or K == 0:
        return np.zeros(R * tiles_per_row(K), np.uint8), np.zeros(0, np.uint32), np.zeros(R, np.uint32)
    return _encode("bn_host_rice_encode_ranks", (_native.nptr(ranks),), R, K, threads)


def encode(exps: np.ndarray, table: np.ndarray, rank: np.ndarray, threads: int = 0) -> RiceEncoded:
    """Encode [R, K] uint8 exponents (any row range of a tensor) with the tensor's rank table."""
    meta, words, roff = encode_ranks(np.asarray(rank, np.uint8)[exps], threads)
    return RiceEncoded(table=table, meta=meta, bits=words, roff=roff)


def encode_words(w: np.ndarray, rank: np.ndarray, threads: int = 0):
    """Encode straight from BF16 words [R, K] (the packer's path: no exponent plane is built)."""
    w = np.ascontiguousarray(w, np.uint16)
    rank = np.ascontiguousarray(rank, np.uint8)
    R, K = w.shape
    if R == 0 or K == 0:
        return np.zeros(R * tiles_per_row(K), np.uint8), np.zeros(0, np.uint32), np.zeros(R, np.uint32)
    return _encode("bn_host_rice_encode", (_native.nptr(w), _native.nptr(rank)), R, K, threads)


def decode_ranks(meta, words, roff, K: int):
    """GPU decode -> (ranks uint8 [R, K], rend uint32 [R]); rend[r] is the word after row r's last
    bit, to be compared with the next row's offset (the contract of the reference's rice_ranks
    kernel, binade/mlx/rice_kernel.py:71-98)."""
    from .cuda import kernels

    ranks, rend = kernels.rice_ranks(kernels.to_device(meta), kernels.to_device(words), kernels.to_device(roff), K)
    return ranks[:, :K].cpu().numpy(), rend.cpu().numpy()


def decode(enc: RiceEncoded, R: int, K: int) -> np.ndarray:
    """Inverse of encode -> [R, K] uint8 exponents; ValueError unless every row ends where the
    next one starts."""
    if enc.meta.size != R * tiles_per_row(K) or enc.roff.size != R:
        raise ValueError(f"{enc.meta.size} tiles and {enc.roff.size} row offsets for {R} x {K}")
    ranks, rend = decode_ranks(enc.meta, enc.bits, enc.roff, K)
    nxt = np.append(enc.roff[1:].astype(np.int64), enc.bits.size)
    if np.any(rend.astype(np.int64) != nxt):
        raise ValueError("bit stream length does not match meta")
    return np.asarray(enc.table)[ranks]
