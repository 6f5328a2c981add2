"""The R4 hook inside a small Llama-shaped decoder (the reference tests its runtime the same
way, tests/test_r4.py:15-54), and from_dense against the file path."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def tiny():
    from binade_b200.cuda.llama import LlamaShape

    return LlamaShape(layers=2, hidden=256, ffn=512, heads=4, kv_heads=2, head_dim=64, vocab=512, max_seq=48)


def test_from_dense_equals_pack_and_transcode():
    from binade_b200 import pack
    from binade_b200.cuda import kernels as ck
    from binade_b200.cuda import r4
    from test_gpu_parity import weights, words

    for shape in ((96, 704), (3, 40, 128), (33, 100)):
        u = weights(np.random.default_rng(sum(shape)), shape)
        a = r4.from_dense(ck.to_device(u).view(torch.bfloat16))
        b = r4.transcode(pack.pack(u))
        for k in ("raw", "codes", "flags", "esc", "row_esc", "table"):
            assert torch.equal(a[k].reshape(-1), b[k].reshape(-1)), k
        assert a["shape"] == tuple(shape)
        assert np.array_equal(words(r4.R4Linear(a).dense()), u)


def test_decoder_r4_matches_bf16_weights_and_graph_matches_eager():
    from binade_b200.cuda.llama import Decoder

    prompt = torch.randint(0, 512, (6,), device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    m = Decoder(tiny(), kind="r4")
    eager, _ = m.generate(prompt, 12, use_graph=False)
    graphed, secs = m.generate(prompt, 12, use_graph=True)
    assert torch.equal(eager, graphed) and secs > 0
    # every R4 linear rebuilds to exactly the BF16 weight the dense model multiplies by
    d = Decoder(tiny(), kind="bf16")
    for a, b in zip(list(m.qkv) + list(m.gate_up) + list(m.o) + list(m.down) + [m.lm_head], list(d.qkv) + list(d.gate_up) + list(d.o) + list(d.down) + [d.lm_head]):
        assert torch.equal(a.dense().reshape(b.w.shape), b.w)
    # the token table is compressed too: lookups return the BF16 rows the dense model reads
    assert torch.equal(m.embed(prompt), d.embed.index_select(0, prompt))
    # same weights, different summation order (documented lane order vs cuBLAS): logits agree
    # to BF16 rounding, not bit for bit
    tok, pos = prompt[:1].clone(), torch.zeros(1, dtype=torch.int64, device="cuda")
    lr, ld = m.step(tok, pos).float(), d.step(tok, pos).float()
    assert torch.allclose(lr, ld, atol=2e-2, rtol=2e-2)
    assert m.linear_bytes() < 0.8 * d.linear_bytes()
