"""R4 runtime on CUDA: format-2 arrays from the file, 4-bit rank codes in GPU memory.

Same roles and names as the reference's binade/mlx/r4.py, on torch:
  transcode(module)   Rice arrays {raw, table, meta, bits, roff} -> R4 dict, on the GPU in one
                      fused pass (reference: transcode + _rank_chunks, r4.py:119-175)
  R4Linear(a)         the linear-layer hook: y = x @ W.T with W decoded inside the kernel
  R4LinearGroup(ms)   projections sharing an input: one launch for all of them at batch 1
  R4Embedding(a)      token rows decoded from an R4 table (r4.py:303-325); as_linear for tied heads
  RiceEmbedding(w)    gather-only table kept as a Rice stream, about 10.7 bits per weight resident
                      (r4.py:328-367)
  convert(model)      swap every BinadeLinear holder for an R4Linear in place (r4.py:375-410)

Row counts: 1..FUSED_MAX_ROWS input rows run the fused decode kernel (weights stream once, fp32
accumulation in the documented lane order; `fused_rows` forces it up to 16 rows); up to
MMA_MAX_ROWS rows run the tensor-core decode GEMM (weights stream once, the hardware's summation
order; the reference's counterpart is its fused GEMM for 1 < M <= 128, r4.py:254-268); more rows
rebuild the BF16 weight with the decode kernel and call torch.matmul, as the reference does for
long prompts (r4.py:288).
"""

from __future__ import annotations

import numpy as np
import torch
from torch import nn

from ..format import TILE
from . import kernels as ck

FUSED_MAX_ROWS = 4  # input rows served by the fused decode kernel in the documented order (15360 x 3840: 37 / 49 / 75 us at 2 / 4 / 8 rows); from 5 rows the tensor-core decode GEMM is faster (46 us)


MMA_MAX_ROWS = 256  # input rows served by the tensor-core decode GEMM (one pass over the weights; 256 is the MMA's widest N); beyond, rebuild + cuBLAS


MMA_MAX_PASSES = 1  # passes of MMA_MAX_ROWS rows that still beat rebuild + cuBLAS (15360 x 3840: 55 us a pass against 44 us for the rebuild: beyond one pass the rebuild wins)


class BinadeLinear(nn.Module):
    """Holder of one packed weight's file arrays (`weight` = dict of raw, table, meta, bits, roff,
    numpy or torch) until `convert` turns it into an R4Linear. It cannot run."""

    def __init__(self, weight: dict):
        super().__init__()
        self.weight = weight

    def forward(self, x):
        raise RuntimeError("packed weights run on the R4 runtime: call binade_b200.cuda.r4.convert(model)")


class BinadeEmbedding(nn.Module):
    """Holder of one packed embedding table's file arrays until `convert` swaps it. gather_only
    marks a table that never enters a matmul; it is then kept in its file coding
    (RiceEmbedding), as the reference does (binade/mlx/slow_linear.py:149-160, r4.py:397-399)."""

    def __init__(self, weight: dict, gather_only: bool = False):
        super().__init__()
        self.weight = weight
        self.gather_only = gather_only

    def forward(self, ids):
        raise RuntimeError("packed tables run on the R4 runtime: call binade_b200.cuda.r4.convert(model)")


def transcode(module) -> dict:
    """R4 arrays for a format-2 or format-1 module (anything with a `.weight` dict, or the dict).
    Rows of K weights, K % 4 == 0 (raw bytes are read four at a time); a last tile with K % 128
    weights is padded with code 0. Raises ValueError if a row's stream does not end where the
    next one starts."""
    w = module.weight if hasattr(module, "weight") else module
    raw = ck.to_device(w["raw"])
    K = raw.shape[-1]
    R = raw.numel() // K if K else 0
    if K % 4:
        raise ValueError(f"R4 needs K % 4 == 0, got {K}")
    T = -(-K // TILE)
    if "bits" not in w:  # format 1: fixed-width codes {raw, table, meta, idx, esc} (reference r4.py:134-140)
        if "idx" not in w:
            raise ValueError("neither format 2 (bits, roff) nor format 1 (idx, esc) arrays")
        f1 = ck.Format1(w["meta"], w["idx"], w["esc"], w["table"], R, K)
        codes, flags, esc, row_esc = f1.to_r4()
        return {"raw": raw.reshape(R, K), "table": f1.table, "codes": codes, "flags": flags, "esc": esc, "row_esc": row_esc, "shape": tuple(raw.shape)}
    meta, bits, roff, table = (ck.to_device(w[k]) for k in ("meta", "bits", "roff", "table"))
    if meta.numel() != R * T or roff.numel() != R:
        raise ValueError(f"{meta.numel()} tiles and {roff.numel()} row offsets for {R} x {K}")
    codes, flags, esc, row_esc, bad = ck.rice_to_r4(meta, bits, roff, table, R, K)
    if bad >= 0:
        raise ValueError(f"Rice stream of row {bad} does not end where the next row starts")
    return {"raw": raw.reshape(R, K), "table": table, "codes": codes, "flags": flags, "esc": esc, "row_esc": row_esc, "shape": tuple(raw.shape)}


def from_dense(w: torch.Tensor) -> dict:
    """R4 arrays straight from a BF16 weight [.., K] already on the GPU (K % 4 == 0), without
    going through a file: exponent histogram -> rank table -> 4-bit codes, flags and escapes with
    torch ops on the device (the histogram alone crosses to the host). Gives the arrays that
    packing the tensor and expanding it (pack.pack + transcode) would give; meant for synthetic
    models and tests, where Rice-encoding billions of weights on the host first serves nothing."""
    from ..format import rank_table

    if w.dtype != torch.bfloat16 or not w.is_cuda:
        raise ValueError("from_dense takes a bfloat16 tensor on a CUDA device")
    shape = tuple(w.shape)
    K = shape[-1]
    if K % 4:
        raise ValueError(f"R4 needs K % 4 == 0, got {K}")
    u = w.contiguous().view(torch.int16).reshape(-1, K)
    R, T = u.shape[0], -(-K // TILE)
    exps = ((u.to(torch.int32) >> 7) & 0xFF).to(torch.uint8)
    raw = (((u.to(torch.int32) >> 8) & 0x80) | (u.to(torch.int32) & 0x7F)).to(torch.uint8)
    hist = torch.bincount(exps.reshape(-1).to(torch.int64), minlength=256).cpu().numpy()
    table, rank = rank_table(hist)
    ranks = ck.to_device(rank)[exps.to(torch.int64)]  # uint8 [R, K]
    del exps
    if K != T * TILE:
        ranks = torch.nn.functional.pad(ranks, (0, T * TILE - K))
    hit = ranks >= 15
    table_t = ck.to_device(table)
    esc = torch.cat([table_t[ranks[hit].to(torch.int64)], torch.zeros(1, dtype=torch.uint8, device=w.device)])
    per_row = hit.sum(dim=1)
    row_esc = (torch.cumsum(per_row, 0) - per_row).to(torch.int32)
    flags = hit.view(R, T, TILE).any(dim=2).to(torch.uint8).reshape(-1)
    q = torch.clamp(ranks, max=15).to(torch.int32).view(R, T * 32, 4)
    codes = (q[..., 0] | (q[..., 1] << 4) | (q[..., 2] << 8) | (q[..., 3] << 12)).to(torch.int16).reshape(-1)
    return {"raw": raw, "table": table_t, "codes": codes, "flags": flags, "esc": esc, "row_esc": row_esc, "shape": shape}


def ulp_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance between two bfloat16 tensors in units in the last place: the difference of their
    positions on the number line of BF16 values (+0 and -0 coincide), as int32."""
    def key(t):
        v = t.contiguous().view(torch.int16).to(torch.int32) & 0xFFFF
        return torch.where(v >= 0x8000, -(v & 0x7FFF), v)

    return (key(a) - key(b)).abs()


def r4_bytes(a: dict) -> int:
    """Bytes a matvec streams: every R4 array (reference: scripts/matvec_bench.py:34-35)."""
    return sum(a[k].numel() * a[k].element_size() for k in ck.R4_KEYS)


class _R4:
    """Shared R4 storage, the fused kernels and the BF16 rebuild."""

    def _init_r4(self, a: dict):
        self._a = a
        self.N, self.K = a["raw"].shape
        self.T = -(-self.K // TILE)
        ck.r4_esc_columns(a)  # derived once per matrix: the batch-1 kernels walk escapes by column
        self._struct = ck.r4_struct(a)  # device addresses of the arrays above, which this object keeps alive

    def _matvec(self, x: torch.Tensor) -> torch.Tensor:
        """x [..., K] holding one row -> [..., N]."""
        return ck.r4_matvec(self._a, x.contiguous(), self.N, self.K, self._struct)

    def _gather(self, x, xi, ei, n: int, rs: int, r0: int = 0, *, split: int | None = None, shape: tuple | None = None):
        """[G, n] outputs (or `shape`): pair g multiplies input row xi[g] of x [.., K] by storage
        rows ei[g] * rs + r0 .. + n. With split, the pair [G, split], [G, n - split]."""
        return ck.r4_gather(self._a, x.contiguous(), xi.to(torch.int32), ei.reshape(-1).to(torch.int32), n, rs, r0, self.K, split, shape)

    def _gather_grouped(self, x, xi, ei, E: int, max_per_expert: int, n: int, rs: int, r0: int = 0, *, split: int | None = None):
        """_gather's outputs with every expert's rows read once for all the slots routed to it
        (bit-identical results); None when the shape is outside the grouped kernel (K % 16)."""
        if self.K % 16 or self.T > 200:
            return None
        return ck.r4_gather_grouped(self._a, x.contiguous(), xi.to(torch.int32), ei.reshape(-1).to(torch.int32), E, max_per_expert, n, rs, r0, self.K, split)

    def dense(self, n: int | None = None, rs: int | None = None, r0: int = 0) -> torch.Tensor:
        """The BF16 weight, rebuilt from R4. With n, rs, r0: rows r0 .. r0 + n - 1 of every block of
        rs storage rows, as [N * n / rs, K]."""
        if n is None:
            return ck.r4_decode(self._a, self.N, self.K).reshape(self._a["shape"])
        return ck.r4_decode(self._a, self.N // rs * n, self.K, n, rs, r0)

    def fused_rows(self, x: torch.Tensor) -> torch.Tensor:
        """x [..., K] with 1..16 rows -> [..., N] through the fused decode kernel, every output in
        the documented summation order (the same bits as the one-row kernel gives row by row)."""
        M = x.numel() // self.K
        return ck.r4_rows(self._a, x.reshape(M, self.K).contiguous(), self.N, self.K).reshape(*x.shape[:-1], self.N)

    def mma_rows(self, x: torch.Tensor, split: int | None = None) -> torch.Tensor:
        """x [..., K] -> [..., N] through the tensor-core decode GEMM, 256 rows a pass (weights
        decoded to BF16 inside the kernel and read once; the sum over K in the hardware's order:
        16 k per MMA step, in order, from zero). split: the K tiles in that many equal slices,
        summed apart and added in fp32; default: what `mirror_cublas` found for this row count,
        else 1."""
        M = x.numel() // self.K
        x2 = x.reshape(M, self.K).contiguous()
        if split is None:
            split = getattr(self, "_cublas_split", {}).get(M, 1)
        if M <= MMA_MAX_ROWS:
            y = ck.r4_mma(self._a, x2, self.N, self.K, split)
        else:  # a pass over the weights per 256 rows: still cheaper than rebuilding them for a few passes
            y = torch.cat([ck.r4_mma(self._a, x2[m0 : m0 + MMA_MAX_ROWS], self.N, self.K, split) for m0 in range(0, M, MMA_MAX_ROWS)])
        return y.reshape(*x.shape[:-1], self.N)

    def mirror_cublas(self, rows=(8, 16, 32, 64, 128, 256), seed: int = 0) -> dict:
        """For each row count M, find the split-K count with which `mma_rows` reproduces, bit for
        bit, this device's BF16 GEMM (`x @ W.T` of torch, i.e. cuBLAS) on the decoded weight, and
        remember it for later `mma_rows` calls of that row count. The reference reads cuBLASLt's
        heuristic and mirrors its split-K schemes (binade/mlx/cublas_plan.py:84-192); here the
        plan is found by trying: on B200 cuBLAS sums 16 k per tensor-core step in order from zero,
        as this kernel does, and for few rows and long K cuts K in two halves whose fp32 sums it
        adds. Returns {M: split, or None when no candidate matches}. Needs the dense weight for
        the comparison (rebuilt once, freed on return)."""
        dense = self.dense().reshape(self.N, self.K)
        g = torch.Generator(device=dense.device).manual_seed(seed)
        found, self._cublas_split = {}, getattr(self, "_cublas_split", {})
        for M in rows:
            x = torch.randn((M, self.K), device=dense.device, generator=g).to(torch.bfloat16)
            want = (x @ dense.T).view(torch.int16)
            found[M] = None
            for split in (1, 2, 3, 4, 6, 8):
                if self.T % split or split * (-(-M // 16) * 16) > 512:
                    continue
                if torch.equal(self.mma_rows(x, split).view(torch.int16), want):
                    found[M] = self._cublas_split[M] = split
                    break
        return found

    def _rows(self, x: torch.Tensor) -> torch.Tensor:
        M = x.numel() // self.K
        if M == 1:
            return self._matvec(x)
        if M <= FUSED_MAX_ROWS:
            return self.fused_rows(x)
        if M <= MMA_MAX_PASSES * MMA_MAX_ROWS and self.K % 8 == 0:
            return self.mma_rows(x)
        return x @ self.dense().reshape(self.N, self.K).T


class R4Linear(nn.Module, _R4):
    def __init__(self, a: dict):
        nn.Module.__init__(self)
        self._init_r4(a)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self._rows(x)


class R4LinearGroup(nn.Module):
    """Projections that share their input (q, k and v of an attention block; gate and up of an
    MLP): forward(x) returns the list of their outputs. One input row goes through a single
    launch for up to four matrices (bn_r4_rows_multi), every output bit-identical to what its own
    R4Linear gives; more rows go module by module. The reference launches one kernel per
    projection (binade/mlx/r4.py:186-192)."""

    def __init__(self, linears):
        super().__init__()
        self.linears = nn.ModuleList(list(linears))
        ks = {m.K for m in self.linears}
        self._group = ck.R4Group([m._struct for m in self.linears], [m.N for m in self.linears], ks.pop()) if len(ks) == 1 and 1 <= len(self.linears) <= 4 else None

    def forward(self, x: torch.Tensor):
        if self._group is not None and x.numel() == self._group.K:
            return self._group(x.contiguous())
        return [m(x) for m in self.linears]


class R4Embedding(nn.Module, _R4):
    """Rows for token ids from an R4 table: one kernel decodes only the looked-up rows, with no
    host synchronisation (reference: R4Embedding, binade/mlx/r4.py:303-325)."""

    def __init__(self, a: dict):
        nn.Module.__init__(self)
        self._init_r4(a)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        flat = ids.reshape(-1).to(device=self._a["raw"].device, dtype=torch.int32)
        return ck.r4_lookup(self._a, flat, self.N, self.K).reshape(*ids.shape, self.K)

    def as_linear(self, x: torch.Tensor) -> torch.Tensor:
        """x @ table.T (a tied output head) through the fused decode kernels."""
        return self._rows(x)


class RiceEmbedding(nn.Module):
    """Gather-only table kept in format 2 (Rice) in GPU memory. A lookup decodes just the rows
    asked for: their stream offsets are read inside the kernel, so ids never visit the host.
    No as_linear: the table never enters a matmul (reference: RiceEmbedding, r4.py:328-367)."""

    def __init__(self, w: dict):
        super().__init__()
        w = w.weight if hasattr(w, "weight") else w
        raw = ck.to_device(w["raw"])
        self.K = raw.shape[-1]
        self.N = raw.numel() // self.K
        self.T = -(-self.K // TILE)
        meta, bits, roff, table = (ck.to_device(w[k]) for k in ("meta", "bits", "roff", "table"))
        if meta.numel() != self.N * self.T or roff.numel() != self.N:
            raise ValueError(f"{meta.numel()} tiles and {roff.numel()} row offsets for {self.N} x {self.K}")
        self._a = {"raw": raw.reshape(self.N, self.K), "table": table, "meta": meta.reshape(-1), "bits": bits, "roff": roff, "shape": tuple(raw.shape)}

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        a = self._a
        flat = ids.reshape(-1).to(device=a["raw"].device, dtype=torch.int32)
        return ck.rice_lookup(a["meta"], a["bits"], a["roff"], a["table"], a["raw"], self.N, self.K, flat).reshape(*ids.shape, self.K)

    def dense(self) -> torch.Tensor:
        """The BF16 table."""
        a = self._a
        return ck.rice_unpack(a["meta"], a["bits"], a["roff"], a["table"], a["raw"], self.N, self.K)[0].reshape(a["shape"])


def convert(model: nn.Module, log=None) -> int:
    """Swap every file-array holder for its runtime counterpart in place: BinadeLinear ->
    R4Linear, BinadeEmbedding -> R4Embedding, or RiceEmbedding for a gather-only table,
    moe.BinadeSwitchGLU -> moe.R4SwitchGLU; returns
    how many were converted (reference: r4.py:375-410). Each holder's file arrays are dropped as
    soon as its runtime arrays exist."""
    from . import moe

    todo = [(parent, name) for parent in model.modules() for name, child in parent.named_children() if isinstance(child, (BinadeLinear, BinadeEmbedding, moe.BinadeSwitchGLU))]
    for i, (parent, name) in enumerate(todo, 1):
        holder = getattr(parent, name)
        if isinstance(holder, moe.BinadeSwitchGLU):  # both expert stacks of a layer (reference r4.py:388-391)
            new = moe.R4SwitchGLU(R4Linear(transcode(holder.gate_up_proj)), R4Linear(transcode(holder.down_proj)), holder._activation)
            setattr(parent, name, new)
            holder.gate_up_proj = holder.down_proj = None
            if log and (i % 50 == 0 or i == len(todo)):
                log(f"R4 transcode {i}/{len(todo)}")
            continue
        if isinstance(holder, BinadeEmbedding):
            new = RiceEmbedding(holder.weight) if holder.gather_only and "bits" in holder.weight else R4Embedding(transcode(holder))
        else:
            new = R4Linear(transcode(holder))
        setattr(parent, name, new)
        holder.weight = None
        if log and (i % 50 == 0 or i == len(todo)):
            log(f"R4 transcode {i}/{len(todo)}")
    return len(todo)


def holders(packed) -> dict:
    """{tensor name: BinadeLinear} for every packed weight of an unpack.PackedModel (or a path to
    a packed directory), file arrays read to host memory."""
    from .. import st
    from ..unpack import PackedModel

    pm = packed if isinstance(packed, PackedModel) else PackedModel(packed)
    out = {}
    for name in pm.packed:
        parts = ("raw", "table", "meta", "bits", "roff") if f"{name}.bits" in pm.infos else ("raw", "table", "meta", "idx", "esc")
        out[name] = BinadeLinear({k: st.read(pm.infos[f"{name}.{k}"]) for k in parts})
    return out
