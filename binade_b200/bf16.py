"""BF16 bit fields. A BF16 word is sign (bit 15), exponent (bits 14..7), mantissa (bits 6..0).

Binade stores `raw = sign << 7 | mantissa` verbatim and compresses only the exponent byte
(same split as the reference's binade/bf16.py:20-41). Inputs may be numpy uint16 arrays or
torch tensors (uint16, int16 or bfloat16, on any device); outputs match the input's kind.
"""

from __future__ import annotations

import numpy as np


def _as_words(w):
    """(kind, int32-valued array of 16-bit patterns)."""
    if isinstance(w, np.ndarray):
        if w.dtype != np.uint16:
            raise TypeError(f"expected uint16 BF16 bit patterns, got {w.dtype}")
        return "np", w
    import torch

    if not isinstance(w, torch.Tensor):
        raise TypeError(f"expected a numpy array or torch tensor, got {type(w)}")
    if w.dtype in (torch.bfloat16, torch.uint16):
        w = w.view(torch.int16)
    if w.dtype != torch.int16:
        raise TypeError(f"expected BF16 bit patterns, got {w.dtype}")
    return "torch", w.to(torch.int32) & 0xFFFF


def exponent(w):
    """BF16 words -> uint8 exponent field."""
    kind, v = _as_words(w)
    e = (v >> 7) & 0xFF
    if kind == "np":
        return e.astype(np.uint8)
    import torch

    return e.to(torch.uint8)


def raw(w):
    """BF16 words -> uint8 `sign << 7 | mantissa`."""
    kind, v = _as_words(w)
    r = ((v >> 8) & 0x80) | (v & 0x7F)
    if kind == "np":
        return r.astype(np.uint8)
    import torch

    return r.to(torch.uint8)


def split(w):
    """(raw, exponent)."""
    return raw(w), exponent(w)


def join(r, e):
    """Inverse of split. numpy in -> uint16 words; torch in -> bfloat16 tensor."""
    if isinstance(r, np.ndarray):
        r16, e16 = r.astype(np.uint16), np.asarray(e).astype(np.uint16)
        return ((r16 & 0x80) << 8) | (e16 << 7) | (r16 & 0x7F)
    import torch

    r32, e32 = r.to(torch.int32), e.to(torch.int32)
    u = ((r32 & 0x80) << 8) | (e32 << 7) | (r32 & 0x7F)
    return u.to(torch.int16).view(torch.bfloat16)  # int32 -> int16 keeps the low 16 bits
