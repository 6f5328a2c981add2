"""Row-sharded R4 linears across the GPUs of one node (one process per GPU, NCCL over NVLink).

Output rows are independent and every row's K-sum stays on one GPU, so sharding by rows keeps
each output bit-identical for any GPU count (splitting K would change the summation order). The
reference is single-device; this module is the multi-GPU form of its linear-layer hook.

  row_range(N, rank, world)        rows [r0, r1) of rank `rank`
  shard_packed(p, rank, world)     format-2 arrays of those rows only (what a rank loads and expands)
  shard_r4(a, rank, world)         the same cut on an R4 dict that is already expanded
  RowShardedLinear(local, N, ...)  y = all_gather(local(x)) over the process group
  RowShardedGroup(locals, Ns, ...) several projections of the same input (q, k, v; gate, up)
                                   with one all-gather for all of them
  gather_all(slices, ...)          one collective for the slices of several groups

  make_exchange(group, max_bytes)  a PushGather, or None when the ranks should stay on NCCL
  PushGather(group, max_bytes)     the all-gather as one kernel of this library over NVLink peer
                                   memory (symmetric buffers from torch.distributed); the sharded
                                   modules take it as `exchange=` in place of the NCCL call

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


class PushGather:
    """All-gather of small slices by peer stores (bn_push_gather): every rank writes its slice
    into every peer's symmetric buffer and the ranks meet on flags, in one kernel launch per rank
    and call. torch.distributed's symmetric memory allocates and maps the buffers (plumbing); the
    kernel is this library's. Needs CUDA ranks of one node with peer access; at most 8 ranks.

        ex = PushGather(group, max_bytes)   # collective: every rank of the group
        out = ex(flat)                      # flat [M, W] on this rank -> [world, M, W]

    Results are views of this object's output buffer: the next call on the same object overwrites
    them (after this rank's readers, in stream order), so a result must be consumed or copied
    before the object is used again. Safe to capture in a
    CUDA graph (the call number lives in device memory).

    A peer that never arrives does not hang the GPU: the kernel's wait is bounded (two seconds
    by default), after which it sets the device status and returns with the output incomplete.
    The kernel cannot tell the host by itself, so call `check()` wherever the host synchronises
    anyway (the end of a generation, after a batch of graph replays): it raises, on every rank,
    if any rank gave up, and retires the object (`gather_rows` then returns None and callers fall
    back to the library collective)."""

    HEADER = 256

    def __init__(self, group=None, max_bytes: int = 1 << 20):
        import ctypes

        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > 8:
            raise ValueError("PushGather serves at most 8 ranks")
        self.cap = (max_bytes + 15) // 16 * 16
        self.area = self.world * self.cap  # one data area: every rank's slices
        dev = torch.device("cuda", torch.cuda.current_device())
        self.out = torch.empty(self.area, dtype=torch.uint8, device=dev)  # where the kernel leaves the gathered slices
        self.buf = symm_mem.empty(self.HEADER + 2 * self.area, dtype=torch.uint8, device=dev)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, group)
        self.peers = (ctypes.c_uint64 * self.world)(*[int(p) for p in self.handle.buffer_ptrs])
        self.counter = torch.zeros(4, dtype=torch.int32, device=dev)  # call number; the three-kernel form also keeps two tickets and the wait's outcome here
        self.group, self.dead = group, False
        torch.cuda.synchronize()
        dist.barrier(group)  # every buffer is zeroed before anyone's first flag arrives

    def check(self) -> None:
        """Raises RuntimeError on every rank if a kernel of this library gave up a wait on any
        rank since the last check (synchronises the device and the group). The object is then
        retired: after a lost exchange the ranks' call numbers may differ."""
        import ctypes

        import torch.distributed as dist

        from .. import _native

        st = ctypes.c_int(0)
        _native.call("cuda", "bn_device_status", ctypes.byref(st))
        flag = torch.tensor([st.value], device=self.out.device, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.group)
        if int(flag.item()):
            self.dead = True
            _native.call("cuda", "bn_device_status_reset")
            raise RuntimeError(f"a bounded wait of the peer-store exchange ran out (device status {int(flag.item()):#x} on some rank): the gathered data is incomplete; this exchange is retired")

    def _push(self, pieces, beside: bool = False):
        """One exchange of 1..8 contiguous device tensors (16-byte aligned, sizes a multiple of
        16 bytes): returns, per piece, the uint8 view [world, bytes] of the gathered slices.
        beside: the three-small-kernels form, for an exchange on a stream of its own."""
        import ctypes

        from .kernels import _call, _p

        sizes = [t.numel() * t.element_size() for t in pieces]
        if sum(sizes) > self.cap:
            raise ValueError(f"slices of {sum(sizes)} bytes exceed the exchange's {self.cap}")
        n = len(pieces)
        ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in pieces])
        lens = (ctypes.c_uint64 * n)(*sizes)
        _call("bn_push_gather_beside" if beside else "bn_push_gather", ctypes.cast(ptrs, ctypes.c_void_p), ctypes.cast(lens, ctypes.c_void_p), n, ctypes.cast(self.peers, ctypes.c_void_p), self.area, _p(self.out), self.rank, self.world, _p(self.counter))
        out, at = [], 0
        for sz in sizes:
            out.append(self.out[at : at + self.world * sz].view(self.world, sz))
            at += self.world * sz
        return out

    @staticmethod
    def _pushable(t: torch.Tensor) -> bool:
        return t.is_contiguous() and t.data_ptr() % 16 == 0 and (t.numel() * t.element_size()) % 16 == 0 and t.numel() > 0

    def gather_rows(self, ys, beside: bool = False):
        """Single-row slices ys[j] [.., w_j] (one row each) of 1..8 projections -> their full
        rows [.., world * w_j], written by the kernel in their final layout: the results are
        views of this rank's buffer, no copy before or after. None if a slice cannot be pushed
        as it is (several rows, unaligned or odd size) or the object is retired: the caller then
        takes another route."""
        if self.dead or not 1 <= len(ys) <= 8 or any(y.numel() != y.shape[-1] or not self._pushable(y) for y in ys):
            return None
        return [g.view(y.dtype).reshape(*y.shape[:-1], self.world * y.shape[-1]) for g, y in zip(self._push(list(ys), beside), ys)]

    def __call__(self, flat: torch.Tensor) -> torch.Tensor:
        if self.dead:
            raise RuntimeError("this exchange was retired after a lost wait")
        flat = flat.contiguous()
        nbytes = flat.numel() * flat.element_size()
        padded = (nbytes + 15) // 16 * 16
        if padded > self.cap:
            raise ValueError(f"slice of {nbytes} bytes exceeds the exchange's {self.cap}")
        if padded != nbytes or flat.data_ptr() % 16:
            stage = torch.zeros(padded, dtype=torch.uint8, device=flat.device)
            stage[:nbytes] = flat.reshape(-1).view(torch.uint8)
            src = stage
        else:
            src = flat
        data = self._push([src])[0][:, :nbytes]
        return data.reshape(self.world, nbytes).view(flat.dtype).view(self.world, *flat.shape)


def make_exchange(group=None, max_bytes: int = 1 << 20):
    """A PushGather for the group, or None (the sharded modules then use the library collective)
    when BINADE_B200_GATHER=nccl, when the ranks are not CUDA ranks, or when any rank could not set
    the symmetric buffers up; the ranks agree on the outcome with one all-reduce, so they never
    end up on different collectives. Collective: every rank of the group calls it."""
    import os
    import sys

    import torch.distributed as dist

    if os.environ.get("BINADE_B200_GATHER", "push") == "nccl" or not torch.cuda.is_available() or dist.get_backend(group) != "nccl":
        return None
    ex, ok = None, 1
    try:
        ex = PushGather(group, max_bytes)
    except Exception as e:  # noqa: BLE001 - any set-up failure means "use the library collective"
        print(f"[binade_b200] peer-store exchange unavailable ({type(e).__name__}: {e}); using NCCL all-gather", file=sys.stderr, flush=True)
        ok = 0
    flag = torch.tensor([ok], device="cuda", dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    return ex if int(flag.item()) == 1 else None


def gather_all(slices, group=None, exchange=None, stream=None, _beside: bool = False):
    """One collective for up to eight single-row slices [.., w_j] of evenly sharded projections:
    returns their full rows [.., world * w_j] in rank order = row order. Through the peer-store
    kernel when an exchange is given and the slices can be pushed as they are, else one library
    all-gather of the slices laid side by side.

    With `stream`, the collective runs there, ordered after the work already queued on the
    current stream, and the current stream goes on without it (the next products overlap the
    exchange). The caller makes whatever reads the results wait for `stream`
    (`torch.cuda.current_stream().wait_stream(stream)`)."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    if world == 1:
        return list(slices)
    if stream is not None:
        stream.wait_stream(torch.cuda.current_stream())
        for y in slices:
            y.record_stream(stream)
        with torch.cuda.stream(stream):
            return gather_all(slices, group, exchange, _beside=True)
    if exchange is not None:
        fast = exchange.gather_rows(list(slices), _beside)
        if fast is not None:
            return fast
    widths = [y.shape[-1] for y in slices]
    flat = torch.cat([y.reshape(1, -1) for y in slices], dim=-1)
    out = _all_gather(flat, world, group, None)  # [world, 1, sum of widths]
    res, c = [], 0
    for y, w in zip(slices, widths):
        res.append(out[:, :, c : c + w].movedim(0, 1).reshape(*y.shape[:-1], world * w))
        c += w
    return res


def _all_gather(flat: torch.Tensor, world: int, group, exchange) -> torch.Tensor:
    """[M, W] on every rank -> [world, M, W], by the peer-store kernel when an exchange is given,
    else by NCCL / gloo."""
    if exchange is not None:
        return exchange(flat)
    import torch.distributed as dist

    out = torch.empty((world * flat.shape[0], flat.shape[1]), dtype=flat.dtype, device=flat.device)
    dist.all_gather_into_tensor(out, flat.contiguous(), group=group)
    return out.view(world, flat.shape[0], flat.shape[1])


class RowShardedLinear(nn.Module):
    """y = x @ W.T with W's rows spread over the ranks of `group`: every rank multiplies by its
    own rows (`local`, e.g. an R4Linear over shard_r4 / a transcoded shard_packed) and the slices
    are gathered with one all-gather, in rank order = row order. Ranks may hold different row
    counts (N % world != 0): slices are then padded to the largest count for the collective."""

    def __init__(self, local, N: int, group=None, exchange=None):
        super().__init__()
        self.local = local
        self.N = N
        self.group = group
        self.exchange = exchange  # a PushGather, or None for the library collective

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist

        world, rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        y = self.local(x)
        if world == 1:
            return y
        if self.exchange is not None and self.N % world == 0:
            fast = self.exchange.gather_rows([y])
            if fast is not None:
                return fast[0]
        counts = [r1 - r0 for r0, r1 in (row_range(self.N, r, world) for r in range(world))]
        width = max(counts)
        if y.shape[-1] != counts[rank]:
            raise ValueError(f"rank {rank} produced {y.shape[-1]} rows, its shard has {counts[rank]}")
        if width != y.shape[-1]:
            y = torch.nn.functional.pad(y, (0, width - y.shape[-1]))
        lead = y.shape[:-1]
        flat = y.reshape(-1, width).contiguous()  # [M, width]
        out = _all_gather(flat, world, self.group, self.exchange)
        if all(c == width for c in counts):
            return out.movedim(0, 1).reshape(*lead, world * width)
        return torch.cat([out[r, :, : counts[r]] for r in range(world)], dim=-1).reshape(*lead, self.N)


class RowShardedGroup(nn.Module):
    """Several row-sharded projections of the same input with ONE collective: every rank runs its
    local modules, lays their output slices side by side, one all-gather moves them, and each
    full output is cut back out in rank order = row order. This is how a decoder layer uses the
    hook (q, k and v share their input, so do gate and up): the small-message latency of the
    collective is paid once per group instead of once per projection. Every N must divide evenly
    over the ranks. forward(x) returns the list of full outputs, bit-identical to what
    RowShardedLinear gives for each projection alone. forward(x, gather=False) returns the local
    slices only: a caller with several groups whose outputs are not needed in between (a layer
    that evaluates q k v, o, gate up, down on given inputs) gathers them all with one collective
    (`gather_all`), paying the small-message latency once."""

    def __init__(self, locals_, Ns, group=None, exchange=None):
        super().__init__()
        self.exchange = exchange
        locals_ = list(locals_)
        self.locals = nn.ModuleList(locals_) if all(isinstance(m, nn.Module) for m in locals_) else locals_
        self.Ns = list(Ns)
        self.group = group
        from . import r4

        # R4 projections of one input run as one launch
        self._fused = r4.R4LinearGroup(locals_) if 1 <= len(locals_) <= 4 and all(isinstance(m, r4.R4Linear) for m in locals_) else None

    def forward(self, x: torch.Tensor, gather: bool = True):
        import torch.distributed as dist

        world = dist.get_world_size(self.group)
        ys = self._fused(x) if self._fused is not None else [m(x) for m in self.locals]
        if world == 1 or not gather:
            return ys
        widths = [N // world for N in self.Ns]
        for y, w, N in zip(ys, widths, self.Ns):
            if N % world or y.shape[-1] != w:
                raise ValueError(f"a projection of {N} rows does not split evenly over {world} ranks (local slice {y.shape[-1]})")
        if self.exchange is not None:
            fast = self.exchange.gather_rows(ys)
            if fast is not None:
                return fast
        lead = ys[0].shape[:-1]
        flat = torch.cat([y.reshape(-1, w) for y, w in zip(ys, widths)], dim=-1)  # [M, sum of widths]
        out = _all_gather(flat, world, self.group, self.exchange)
        res, c = [], 0
        for w, N in zip(widths, self.Ns):
            res.append(out[:, :, c : c + w].movedim(0, 1).reshape(*lead, N))
            c += w
        return res
