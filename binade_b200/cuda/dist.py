"""Row-sharded R4 linears across the GPUs of one node (one process per GPU, NCCL over NVLink).

Output rows are independent and every row's K-sum stays on one GPU, so sharding by rows keeps
each output bit-identical for any GPU count (splitting K would change the summation order). The
reference is single-device; this module is the multi-GPU form of its linear-layer hook.

  row_range(N, rank, world)        rows [r0, r1) of rank `rank`
  shard_packed(p, rank, world)     format-2 arrays of those rows only (what a rank loads and expands)
  shard_r4(a, rank, world)         the same cut on an R4 dict that is already expanded
  RowShardedLinear(local, N, ...)  y = all_gather(local(x)) over the process group

The cuts are pure index arithmetic on numpy arrays or torch tensors of any device; only
RowShardedLinear.forward touches a process group.
"""

from __future__ import annotations

import numpy as np
import torch
from torch import nn

from ..format import TILE


def row_range(N: int, rank: int, world: int) -> tuple[int, int]:
    """Even split; the first N % world ranks hold one row more."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(N, world)
    r0 = rank * base + min(rank, extra)
    return r0, r0 + base + (1 if rank < extra else 0)


def shard_packed(p: dict, rank: int, world: int) -> dict:
    """Rows of rank `rank` from {"raw", "table", "meta", "bits", "roff"[, "shape"]} (numpy).
    Rows start on word boundaries and carry their own offset, so a shard is a slice of every
    array with `roff` rebased to the slice of `bits` it keeps."""
    raw = np.asarray(p["raw"])
    K = raw.shape[-1]
    raw2 = raw.reshape(-1, K)
    R, T = raw2.shape[0], -(-K // TILE)
    r0, r1 = row_range(R, rank, world)
    roff = np.asarray(p["roff"])
    w0 = int(roff[r0]) if r0 < R else int(np.asarray(p["bits"]).size)
    w1 = int(roff[r1]) if r1 < R else int(np.asarray(p["bits"]).size)
    return {
        "raw": raw2[r0:r1],
        "table": p["table"],
        "meta": np.asarray(p["meta"])[r0 * T : r1 * T],
        "bits": np.asarray(p["bits"])[w0:w1],
        "roff": (roff[r0:r1].astype(np.int64) - w0).astype(np.uint32),
        "shape": (r1 - r0, K),
    }


def shard_r4(a: dict, rank: int, world: int) -> dict:
    """Rows of rank `rank` from an R4 dict (torch tensors, any device). `row_esc` is rebased to the
    shard's own escape bytes, which keep their closing 0."""
    N, K = a["raw"].shape
    T = -(-K // TILE)
    r0, r1 = row_range(N, rank, world)
    row_esc = a["row_esc"].to(torch.int64) & 0xFFFFFFFF
    n_esc = a["esc"].numel() - 1
    e0 = int(row_esc[r0]) if r0 < N else n_esc
    e1 = int(row_esc[r1]) if r1 < N else n_esc
    esc = torch.cat([a["esc"][e0:e1], torch.zeros(1, dtype=a["esc"].dtype, device=a["esc"].device)])
    return {
        "raw": a["raw"][r0:r1].contiguous(),
        "table": a["table"],
        "codes": a["codes"][r0 * T * 32 : r1 * T * 32].contiguous(),
        "flags": a["flags"][r0 * T : r1 * T].contiguous(),
        "esc": esc,
        "row_esc": (row_esc[r0:r1] - e0).to(torch.int32),
        "shape": (r1 - r0, K),
    }


class RowShardedLinear(nn.Module):
    """y = x @ W.T with W's rows spread over the ranks of `group`: every rank multiplies by its
    own rows (`local`, e.g. an R4Linear over shard_r4 / a transcoded shard_packed) and the slices
    are gathered with one all-gather, in rank order = row order. Ranks may hold different row
    counts (N % world != 0): slices are then padded to the largest count for the collective."""

    def __init__(self, local, N: int, group=None):
        super().__init__()
        self.local = local
        self.N = N
        self.group = group

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist

        world, rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        y = self.local(x)
        if world == 1:
            return y
        counts = [r1 - r0 for r0, r1 in (row_range(self.N, r, world) for r in range(world))]
        width = max(counts)
        if y.shape[-1] != counts[rank]:
            raise ValueError(f"rank {rank} produced {y.shape[-1]} rows, its shard has {counts[rank]}")
        if width != y.shape[-1]:
            y = torch.nn.functional.pad(y, (0, width - y.shape[-1]))
        lead = y.shape[:-1]
        flat = y.reshape(-1, width).contiguous()  # [M, width]
        out = torch.empty((world * flat.shape[0], width), dtype=y.dtype, device=y.device)
        dist.all_gather_into_tensor(out, flat, group=self.group)
        out = out.view(world, flat.shape[0], width)
        if all(c == width for c in counts):
            return out.movedim(0, 1).reshape(*lead, world * width)
        return torch.cat([out[r, :, : counts[r]] for r in range(world)], dim=-1).reshape(*lead, self.N)
