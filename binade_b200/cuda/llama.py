"""A Llama-shaped decoder whose linear layers are the R4 hook: the smallest model harness that
exercises the runtime the way the reference's own tests do with a tiny Llama
(tests/test_r4.py:15-54), and the synthetic 8B-class model of the decode benchmark.

Batch-1 greedy decoding with a static KV cache; one decode step is capturable in a CUDA graph
(token and position live in device tensors). Linear layers are built by a factory, so the same
model runs on R4Linear (fused decode), on plain BF16 weights (cuBLAS) or on RowShardedLinear over
several GPUs. With `world` > 1 every linear is sharded by output rows: a rank owns n_heads/world
query heads with their KV heads and FFN/world rows of gate and up, attention and SwiGLU stay
local, and four all-gathers per layer (attention output, o_proj, SwiGLU output, down_proj) plus
one for the logits rebuild the full vectors, in row order, so outputs do not depend on the GPU
count. The all-gathers are this library's peer-store kernel (dist.PushGather), or NCCL with
BINADE_B200_GATHER=nccl.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
from torch import nn

from . import r4
from .dist import RowShardedLinear, make_exchange, row_range


@dataclass
class LlamaShape:
    layers: int = 32
    hidden: int = 4096
    ffn: int = 14336
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    vocab: int = 128256
    max_seq: int = 320
    rope_theta: float = 500000.0
    eps: float = 1e-5


class DenseLinear(nn.Module):
    """BF16 weight [N, K] through torch (cuBLAS): the baseline the R4 hook is compared with."""

    def __init__(self, w: torch.Tensor):
        super().__init__()
        self.w = w

    def forward(self, x):
        return torch.nn.functional.linear(x, self.w)


def synthetic_weight(rows: int, cols: int, seed: int, device) -> torch.Tensor:
    g = torch.Generator(device=device).manual_seed(seed)
    return (torch.randn((rows, cols), generator=g, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16)


class Decoder(nn.Module):
    def __init__(self, shape: LlamaShape, kind: str = "r4", rank: int = 0, world: int = 1, group=None, device="cuda", seed: int = 0):
        """kind: "r4" (R4Linear over from_dense) or "bf16" (DenseLinear). Weights are N(0, 0.02)
        from fixed seeds, generated whole on every rank and cut to the rank's rows."""
        super().__init__()
        s = self.shape = shape
        if s.heads % world or s.kv_heads % world or s.ffn % world or s.hidden % world or s.vocab % world:
            raise ValueError(f"world {world} does not divide heads, kv_heads, ffn, hidden and vocab")
        self.rank, self.world, self.group, self.seed = rank, world, group, seed
        dev = torch.device(device)
        self.hq, self.hkv = s.heads // world, s.kv_heads // world
        d = s.head_dim

        # the all-gathers go through this library's peer-store kernel (one shared buffer: every
        # gathered vector is consumed before the next exchange in stream order);
        # BINADE_B200_GATHER=nccl keeps them on the library collective
        self.exchange = make_exchange(group, max_bytes=2 * max(s.vocab, s.ffn, s.heads * d, s.hidden) // world + 64) if world > 1 and dev.type == "cuda" else None

        def lin(w_rows: torch.Tensor, n_total: int):
            local = r4.R4Linear(r4.from_dense(w_rows)) if kind == "r4" else DenseLinear(w_rows)
            return RowShardedLinear(local, n_total, group, exchange=self.exchange) if world > 1 else local

        def rows_of(w, count):  # this rank's share of `count` leading-dim rows
            r0, r1 = row_range(count, rank, world)
            return w[r0:r1]

        emb = synthetic_weight(s.vocab, s.hidden, seed + 1, dev)
        self.embed = r4.R4Embedding(r4.from_dense(emb)) if kind == "r4" else emb  # whole table on every rank
        del emb
        self.qkv, self.o, self.gate_up, self.down, self.norm1, self.norm2 = nn.ModuleList(), nn.ModuleList(), nn.ModuleList(), nn.ModuleList(), [], []
        for l in range(s.layers):
            base = seed + 100 * (l + 1)
            wq = synthetic_weight(s.heads * d, s.hidden, base + 1, dev)
            wk = synthetic_weight(s.kv_heads * d, s.hidden, base + 2, dev)
            wv = synthetic_weight(s.kv_heads * d, s.hidden, base + 3, dev)
            # q, k and v rows of this rank's heads as one matrix: one launch instead of three
            # (each output keeps its own row, so fusing rows does not touch any sum)
            local_qkv = torch.cat([rows_of(wq, s.heads * d), rows_of(wk, s.kv_heads * d), rows_of(wv, s.kv_heads * d)])
            self.qkv.append(r4.R4Linear(r4.from_dense(local_qkv)) if kind == "r4" else DenseLinear(local_qkv))
            del wq, wk, wv, local_qkv
            self.o.append(lin(rows_of(synthetic_weight(s.hidden, s.heads * d, base + 4, dev), s.hidden), s.hidden))
            wg = synthetic_weight(s.ffn, s.hidden, base + 5, dev)
            wu = synthetic_weight(s.ffn, s.hidden, base + 6, dev)
            local_gu = torch.cat([rows_of(wg, s.ffn), rows_of(wu, s.ffn)])
            self.gate_up.append(r4.R4Linear(r4.from_dense(local_gu)) if kind == "r4" else DenseLinear(local_gu))
            del wg, wu, local_gu
            self.down.append(lin(rows_of(synthetic_weight(s.hidden, s.ffn, base + 7, dev), s.hidden), s.hidden))
            self.norm1.append(torch.ones(s.hidden, dtype=torch.bfloat16, device=dev))
            self.norm2.append(torch.ones(s.hidden, dtype=torch.bfloat16, device=dev))
        self.norm_f = torch.ones(s.hidden, dtype=torch.bfloat16, device=dev)
        self.lm_head = lin(rows_of(synthetic_weight(s.vocab, s.hidden, seed + 2, dev), s.vocab), s.vocab)
        self.k_cache = torch.zeros((s.layers, self.hkv, s.max_seq, d), dtype=torch.bfloat16, device=dev)
        self.v_cache = torch.zeros_like(self.k_cache)
        inv = 1.0 / (s.rope_theta ** (torch.arange(0, d, 2, device=dev, dtype=torch.float32) / d))
        ang = torch.arange(s.max_seq, device=dev, dtype=torch.float32)[:, None] * inv[None, :]
        self.cos, self.sin = torch.cos(ang), torch.sin(ang)  # [max_seq, d/2]
        self.positions = torch.arange(s.max_seq, device=dev)

    def _sources(self):
        """(module, source weight) for every linear of this rank, weights regenerated one at a
        time from the construction seeds."""
        s, d, dev = self.shape, self.shape.head_dim, self.k_cache.device
        rows_of = lambda w, count: w[slice(*row_range(count, self.rank, self.world))]
        local = lambda m: m.local if isinstance(m, RowShardedLinear) else m
        for l in range(s.layers):
            base = self.seed + 100 * (l + 1)
            wq, wk, wv = (synthetic_weight(n, s.hidden, base + j, dev) for j, n in ((1, s.heads * d), (2, s.kv_heads * d), (3, s.kv_heads * d)))
            yield self.qkv[l], torch.cat([rows_of(wq, s.heads * d), rows_of(wk, s.kv_heads * d), rows_of(wv, s.kv_heads * d)])
            yield local(self.o[l]), rows_of(synthetic_weight(s.hidden, s.heads * d, base + 4, dev), s.hidden)
            yield self.gate_up[l], torch.cat([rows_of(synthetic_weight(s.ffn, s.hidden, base + 5, dev), s.ffn), rows_of(synthetic_weight(s.ffn, s.hidden, base + 6, dev), s.ffn)])
            yield local(self.down[l]), rows_of(synthetic_weight(s.hidden, s.ffn, base + 7, dev), s.hidden)
        yield local(self.lm_head), rows_of(synthetic_weight(s.vocab, s.hidden, self.seed + 2, dev), s.vocab)

    @torch.no_grad()
    def self_check(self) -> dict:
        """For a model on R4 weights: every linear's dense decode must equal its source weight
        bit for bit (raises otherwise), and one decode step (token 0 at position 0) is run with
        every linear's output compared with an fp32 product of the same weights: returns the
        number of linears checked and the largest deviation in BF16 units in the last place
        (the sums differ from fp32 only by their order, so a few ulps at most)."""
        checked, worst = 0, 0
        hooks = []

        def compare(module, inputs, output):
            nonlocal worst
            ref = (inputs[0].reshape(-1, module.K).float() @ module.dense().reshape(module.N, module.K).float().T).to(torch.bfloat16)
            worst = max(worst, int(r4.ulp_distance(output.reshape(ref.shape), ref).max().item()))

        for m, w in self._sources():
            if not isinstance(m, r4.R4Linear):
                return {"linears": 0, "note": "not an R4 model"}
            if not torch.equal(m.dense().reshape(w.shape).view(torch.int16), w.view(torch.int16)):
                raise RuntimeError("an R4 linear does not decode to its source weight")
            checked += 1
            hooks.append(m.register_forward_hook(compare))
            del w
        dev = self.k_cache.device
        self.step(torch.zeros(1, dtype=torch.int64, device=dev), torch.zeros(1, dtype=torch.int64, device=dev))
        for h in hooks:
            h.remove()
        self.k_cache.zero_(), self.v_cache.zero_()
        return {"linears_decoding_to_their_source": checked, "max_ulp_vs_fp32_product_step0": worst}

    def linear_bytes(self) -> int:
        """Weight bytes one decode step streams on this rank (R4 arrays or BF16 words)."""
        total = 0
        for m in list(self.qkv) + list(self.o) + list(self.gate_up) + list(self.down) + [self.lm_head]:
            m = m.local if isinstance(m, RowShardedLinear) else m
            total += r4.r4_bytes(m._a) if isinstance(m, r4.R4Linear) else m.w.numel() * 2
        return total

    def _gather(self, y: torch.Tensor, n_total: int) -> torch.Tensor:
        """All-gather a local slice [.., n_total / world] into the full vector (row order)."""
        if self.world == 1:
            return y
        if self.exchange is not None and not self.exchange.dead:
            fast = self.exchange.gather_rows([y.reshape(1, -1)])
            return fast[0] if fast is not None else self.exchange(y.reshape(1, -1)).reshape(1, n_total)
        import torch.distributed as dist

        out = torch.empty((self.world, y.shape[-1]), dtype=y.dtype, device=y.device)
        dist.all_gather_into_tensor(out, y.reshape(1, -1).contiguous(), group=self.group)
        return out.reshape(1, n_total)

    @staticmethod
    def _rope(t: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        """t [heads, d] rotated by the position's cos / sin [1, d/2] (fp32 arithmetic)."""
        tf = t.float()
        a, b = tf[:, : t.shape[1] // 2], tf[:, t.shape[1] // 2 :]
        return torch.cat([a * cos - b * sin, a * sin + b * cos], dim=1).to(t.dtype)

    def step(self, token: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        """One decode step: token, pos are device int64 tensors of one element -> logits [1, vocab].
        The glue between the linear layers is kept to few kernels (it is launch-bound at batch 1):
        the position's rotation is looked up once per step, q and k rotate together, attention is
        one fused scaled-dot-product call over the static cache with a position mask."""
        s, d = self.shape, self.shape.head_dim
        x = self.embed(token) if isinstance(self.embed, r4.R4Embedding) else self.embed.index_select(0, token)  # [1, hidden]
        mask = (self.positions <= pos)[None, None, None, :]  # [1, 1, 1, max_seq]
        cos, sin = self.cos.index_select(0, pos), self.sin.index_select(0, pos)  # [1, d/2]
        nqk = self.hq + self.hkv
        for l in range(s.layers):
            h = torch.nn.functional.rms_norm(x, (s.hidden,), self.norm1[l], s.eps)
            qkv = self.qkv[l](h)[0]
            qk = self._rope(qkv[: nqk * d].view(nqk, d), cos, sin)
            v = qkv[nqk * d :].view(self.hkv, d)
            self.k_cache[l].index_copy_(1, pos, qk[self.hq :, None, :])
            self.v_cache[l].index_copy_(1, pos, v[:, None, :])
            attn = torch.nn.functional.scaled_dot_product_attention(qk[None, : self.hq, None, :], self.k_cache[l][None], self.v_cache[l][None], attn_mask=mask, enable_gqa=True)  # [1, hq, 1, d]
            x = x + self.o[l](self._gather(attn.reshape(1, self.hq * d), s.heads * d))
            h = torch.nn.functional.rms_norm(x, (s.hidden,), self.norm2[l], s.eps)
            gu = self.gate_up[l](h)[0]
            half = gu.shape[0] // 2
            act = (torch.nn.functional.silu(gu[:half].float()) * gu[half:].float()).to(torch.bfloat16)
            x = x + self.down[l](self._gather(act[None, :], s.ffn))
        return self.lm_head(torch.nn.functional.rms_norm(x, (s.hidden,), self.norm_f, s.eps))

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, n_new: int, use_graph: bool = True):
        """Greedy decoding. prompt: int64 [P] on the device. Returns (tokens int64 [n_new],
        seconds spent on the n_new generated tokens, measured with CUDA events)."""
        P = prompt.numel()
        if P + n_new > self.shape.max_seq:
            raise ValueError("prompt + new tokens exceed max_seq")
        token, pos = prompt[:1].clone(), torch.zeros(1, dtype=torch.int64, device=prompt.device)
        out = torch.zeros(n_new, dtype=torch.int64, device=prompt.device)
        nxt = torch.zeros(1, dtype=torch.int64, device=prompt.device)

        def one():
            logits = self.step(token, pos)
            nxt.copy_(torch.argmax(logits[0].float(), dim=-1, keepdim=True))  # ties: lowest index
            pos.add_(1)

        graph = None
        if use_graph:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                one()  # warm-up outside capture (also sets up lazy state)
                side.synchronize()
                pos.zero_()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    one()
            torch.cuda.synchronize()
            pos.zero_()
        run = graph.replay if graph else one
        for i in range(P):  # the prompt, one token at a time through the same step
            token.copy_(prompt[i : i + 1])
            run()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n_new):
            token.copy_(nxt)
            out[i : i + 1].copy_(nxt)
            run()
        e1.record()
        torch.cuda.synchronize()
        if self.exchange is not None:
            self.exchange.check()  # a peer that never arrived: raise instead of returning tokens from stale vectors
        return out, e0.elapsed_time(e1) / 1e3
