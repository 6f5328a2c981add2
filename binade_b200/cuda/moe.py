"""Mixture-of-experts expert path on R4 weights (reference: binade/mlx/moe.py).

Expert weights are stored fused, as the reference keeps them: gate_up [E * 2n, D] (gate rows
0..n-1, up rows n..2n-1 of every expert) and down [E * D, n]; an expert is a row range, selected
inside the kernel by `ei[g] * rows_per_expert`.

  R4SwitchGLU(gate_up, down, activation)   y[.., k, D] = down_e(act(up_e x, gate_e x)) for the k
                                           experts `indices[.., k]` of every token, one fused
                                           gather launch for gate+up and one for down
  BinadeSwitchGLU(gate_up, down)           holder of the packed stacks until r4.convert
  ExpertParallelGLU(local, E, rank, world)  experts and tokens spread over the ranks of a process
                                           group: an all-to-all brings every slot's input row
                                           to the rank that owns its expert, a second one
                                           takes the outputs back

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


class BinadeSwitchGLU(nn.Module):
    """Holder of one layer's packed expert stacks until `r4.convert` swaps it for an R4SwitchGLU
    (reference: BinadeSwitchGLU, binade/mlx/moe.py:29-52). gate_up_proj / down_proj: dicts of
    file arrays {raw, table, meta, bits, roff} (or format 1), raw shaped [E, 2n, D] and
    [E, D, n]. It cannot run."""

    def __init__(self, gate_up_proj: dict, down_proj: dict, activation=swiglu):
        super().__init__()
        self.gate_up_proj, self.down_proj, self._activation = gate_up_proj, down_proj, activation

    def forward(self, x, indices):
        raise RuntimeError("packed experts run on the R4 runtime: call binade_b200.cuda.r4.convert(model)")


class ExpertParallelGLU(nn.Module):
    """Experts partitioned over the ranks of a process group, tokens too: rank r owns experts
    [r * E/world, (r + 1) * E/world) and brings its own share of the batch. One forward is a
    dispatch, the local expert path, and a combine:

      dispatch  every (token, expert) slot of this rank's tokens travels to the rank that owns
                its expert: one all-to-all of fixed-size chunks. A chunk holds `cap` input rows
                (cap = this rank's slot count, the most one peer can get from it) followed by
                the slots' local expert ids, padding slots marked NO_EXPERT, so the input rows
                and their ids share one collective and no count crosses the host.
      compute   `local_slots(x_rows, xi, ei_local) -> [slots, D]` on what arrived (the `.slots`
                of an R4SwitchGLU over this rank's experts); padding slots are skipped inside
                the kernels, so a rank streams only the experts really routed to it.
      combine   the slot outputs go back the way they came (one all-to-all) and are put in their
                slots' places.

    Every rank must bring the same number of tokens (pad with tokens routed to NO_EXPERT slots
    if need be: indices < 0). A slot is computed by exactly one rank with the single-GPU kernels,
    so outputs are bit-identical to R4SwitchGLU on one GPU."""

    def __init__(self, local_slots, E: int, D: int, rank: int, world: int, group=None):
        super().__init__()
        if E % world:
            raise ValueError(f"{E} experts do not split over {world} ranks")
        self.local_slots, self.E, self.D, self.rank, self.world, self.group = local_slots, E, D, rank, world, group
        self.per = E // world

    def forward(self, x: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
        """x [tokens, D] and indices [tokens, k] of this rank's tokens -> [tokens, k, D]."""
        import torch.distributed as dist

        from .kernels import NO_EXPERT

        k, D, W = indices.shape[-1], self.D, self.world
        flat = x.reshape(-1, D)
        ei = indices.reshape(-1).to(torch.int64)
        S = ei.numel()  # this rank's slots; also the capacity of a chunk
        dev = x.device
        xi = torch.arange(S, device=dev) // k
        real = ei >= 0
        owner = torch.where(real, ei // self.per, torch.full_like(ei, W))  # padding tokens: no owner
        # place of each slot in its owner's chunk: its rank among this rank's slots of that owner
        order = torch.argsort(owner, stable=True)
        counts = torch.zeros(W + 1, dtype=torch.int64, device=dev).scatter_add_(0, owner, torch.ones_like(owner))
        start = torch.cumsum(counts, 0) - counts
        within = torch.empty_like(order)
        within[order] = torch.arange(S, device=dev) - start[owner[order]]
        # a chunk: S input rows, then the ids in as many rows as S int32 values need. Padding
        # slots go to a spare chunk that is not sent: every index below is fixed-shape, so the
        # whole forward can be captured in a CUDA graph
        id_rows = -(-4 * S // (2 * D))
        rows = S + id_rows
        stage = torch.zeros((W + 1, rows, D), dtype=torch.bfloat16, device=dev)
        ids = torch.full((W + 1, id_rows * D // 2), NO_EXPERT, dtype=torch.int32, device=dev)
        stage[owner, within] = flat[xi]
        ids[owner, within] = torch.where(real, ei - owner * self.per, torch.full_like(ei, NO_EXPERT)).to(torch.int32)
        stage[:, S:] = ids.view(torch.bfloat16).view(W + 1, id_rows, D)
        send = stage[:W]
        if W > 1:
            recv = torch.empty_like(send)
            dist.all_to_all_single(recv.view(W * rows, D), send.reshape(W * rows, D), group=self.group)
        else:
            recv = send
        # what arrived: W chunks of S slots each; slot j of chunk p reads input row p * rows + j
        got_ids = recv[:, S:].reshape(W, -1).view(torch.int32)[:, :S].reshape(-1)
        got_xi = (torch.arange(W, device=dev)[:, None] * rows + torch.arange(S, device=dev)[None, :]).reshape(-1).to(torch.int32)
        out = self.local_slots(recv.reshape(W * rows, D), got_xi, got_ids)  # [W * S, D]; rows of padding slots are garbage
        if W > 1:
            back = torch.empty_like(out)
            dist.all_to_all_single(back, out.contiguous(), group=self.group)
        else:
            back = out
        back = torch.cat([back.view(W, S, D), torch.zeros((1, S, D), dtype=back.dtype, device=dev)])  # chunk W: zeros for padding slots
        y = back[owner, within]
        return y.reshape(*indices.shape, D)
