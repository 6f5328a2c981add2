"""Mixture-of-experts expert path on R4 weights (reference: binade/mlx/moe.py).

Expert weights are stored fused, as the reference keeps them: gate_up [E * 2n, D] (gate rows
0..n-1, up rows n..2n-1 of every expert) and down [E * D, n]; an expert is a row range, selected
inside the kernel by `ei[g] * rows_per_expert`.

  R4SwitchGLU(gate_up, down, activation)   y[.., k, D] = down_e(act(up_e x, gate_e x)) for the k
                                           experts `indices[.., k]` of every token, one fused
                                           gather launch for gate+up and one for down
  ExpertParallelGLU(local, E, rank, world)  experts spread over the ranks of a process group:
                                           every rank runs the slots whose expert it owns and
                                           the slot outputs travel back with one all-to-all

Router softmax / top-k and the weighted sum over the k experts stay with the caller, as in the
reference (mlx-lm's SwitchGLU contract).
"""

from __future__ import annotations

import torch
from torch import nn


def swiglu(up: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up in fp32, rounded once to BF16 (the activation of Gemma/Llama style MoE)."""
    return (torch.nn.functional.silu(gate.float()) * up.float()).to(torch.bfloat16)


class R4SwitchGLU(nn.Module):
    def __init__(self, gate_up, down, activation=swiglu):
        """gate_up, down: R4Linear over [E * 2n, D] and [E * D, n] rows."""
        super().__init__()
        self._gu, self._down, self._activation = gate_up, down, activation
        shape_gu, shape_dn = gate_up._a["shape"], down._a["shape"]
        self.E = shape_gu[0] if len(shape_gu) == 3 else None
        if self.E is None:
            raise ValueError("gate_up must keep its [E, 2n, D] shape")
        self.n, self.D = shape_gu[1] // 2, shape_dn[1]

    GROUP_MIN_SLOTS = 2  # from this many slots per expert on average, group the slots by expert

    def slots(self, x: torch.Tensor, xi: torch.Tensor, ei: torch.Tensor, max_per_expert: int | None = None) -> torch.Tensor:
        """[G, D] outputs of G (token row xi[g], expert ei[g]) slots; x [tokens, D]. With more
        slots than experts (a batch of tokens), the slots are grouped by expert so that every
        active expert's weights are read once (same bits as slot by slot); max_per_expert bounds
        the slots of one expert (default: the token count, right when a token names an expert at
        most once, as top-k routing does)."""
        n, G = self.n, ei.numel()
        rows = torch.arange(G, dtype=torch.int32, device=x.device)
        if G >= self.GROUP_MIN_SLOTS * self.E:
            cap = max_per_expert or x.shape[0]
            gu = self._gu._gather_grouped(x, xi, ei, self.E, cap, 2 * n, 2 * n, split=n)
            if gu is not None:
                h = self._activation(gu[1], gu[0])
                out = self._down._gather_grouped(h, rows, ei, self.E, cap, self.D, self.D)
                if out is not None:
                    return out
        gate, up = self._gu._gather(x, xi, ei, 2 * n, 2 * n, split=n)
        h = self._activation(up, gate)
        return self._down._gather(h, rows, ei, self.D, self.D)

    def forward(self, x: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
        """x [..., D], indices [..., k] -> [..., k, D]."""
        k = indices.shape[-1]
        flat = x.reshape(-1, x.shape[-1])
        ei = indices.reshape(-1).to(torch.int32)
        xi = torch.arange(ei.numel(), dtype=torch.int32, device=x.device) // k
        return self.slots(flat, xi, ei).reshape(*indices.shape, self.D)


class ExpertParallelGLU(nn.Module):
    """Experts partitioned over ranks: rank r owns experts [r * E/world, (r+1) * E/world). Every
    rank sees the same tokens and indices (as in tensor-parallel decoding) and computes only the
    slots whose expert it owns, with `local_slots(x, xi, ei_local) -> [G_local, D]` (the `.slots`
    of an R4SwitchGLU over its own experts). Every rank needs every slot's output, so each rank
    sends the slots it computed to all ranks in one all-to-all of fixed-capacity buffers (capacity
    = the number of slots: no count exchange, no host sync) and scatters what it receives to the
    slots' positions. A slot is computed by exactly one rank, so the result does not depend on the
    number of ranks."""

    def __init__(self, local_slots, E: int, D: int, rank: int, world: int, group=None):
        super().__init__()
        if E % world:
            raise ValueError(f"{E} experts do not split over {world} ranks")
        self.local_slots, self.E, self.D, self.rank, self.world, self.group = local_slots, E, D, rank, world, group
        self.per = E // world

    def forward(self, x: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist

        k = indices.shape[-1]
        flat = x.reshape(-1, x.shape[-1])
        ei = indices.reshape(-1).to(torch.int64)
        G = ei.numel()
        xi = torch.arange(G, dtype=torch.int32, device=x.device) // k
        owner = ei // self.per
        mine = owner == self.rank
        # this rank's slots first (stable order), padded with slot 0 of expert 0: fixed shapes
        order = torch.argsort((~mine).to(torch.int8), stable=True)
        n_mine = mine.sum()
        sel_ei = torch.where(torch.arange(G, device=x.device) < n_mine, ei[order] - self.rank * self.per, torch.zeros_like(ei)).to(torch.int32)
        out = self.local_slots(flat, xi[order], sel_ei)  # [G, D]; rows >= n_mine are padding
        if self.world == 1:
            y = torch.empty_like(out)
            y[order] = out
            return y.reshape(*indices.shape, self.D)
        # all-to-all: every rank sends (its slot outputs, their slot numbers, its count) to everyone
        send = out[None].expand(self.world, G, self.D).contiguous()
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv.view(self.world * G, self.D), send.view(self.world * G, self.D), group=self.group)
        meta_send = torch.cat([order.to(torch.int64), n_mine.reshape(1).to(torch.int64)])[None].expand(self.world, G + 1).contiguous()
        meta_recv = torch.empty_like(meta_send)
        dist.all_to_all_single(meta_recv.view(-1), meta_send.view(-1), group=self.group)
        y = torch.zeros((G + 1, self.D), dtype=out.dtype, device=out.device)  # row G swallows padding
        for r in range(self.world):
            pos, cnt = meta_recv[r, :G], meta_recv[r, G]
            dst = torch.where(torch.arange(G, device=x.device) < cnt, pos, torch.full_like(pos, G))
            y.index_copy_(0, dst, recv[r])
        return y[:G].reshape(*indices.shape, self.D)
