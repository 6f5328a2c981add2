"""Generate the golden vectors under tests/golden by running the REFERENCE's own numpy code.

    python tests/golden/make_golden.py /path/to/reference/checkout

Only runs where a checkout of GuyShafir/binade (v0.1.2) is available; the vectors it writes are
committed, so tests never need the checkout. Inputs come from seeded numpy generators; outputs
are whatever the reference computes for them:

  codec_cases.npz   exponent planes [R,K] -> rank table, Rice meta/bits/roff (binade/rice.py,
                    binade/format.py) and the decoder's ranks and row ends
  config1_small.npz a BF16 tensor with the benchmark's value distribution -> split + Rice parts
  r4_layout.npz     the R4 arrays the reference's numpy statement of the layout builds
                    (binade/mlx/kernel.py R4Matrix.__init__, K % 128 == 0), via its format-1 codec
  format1.npz       format-1 encode output (binade/format.py) for the same tensors
  packed_model/     a tiny model packed by binade.pack.pack_model (format 2): the safetensors
                    file, byte for byte, plus the source tensors

The reference's mlx import is satisfied by a stub whose array() is numpy.asarray: none of the
functions used here touches a GPU.
"""

import hashlib
import json
import sys
import types
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def _stub_mlx():
    mx = types.ModuleType("mlx.core")
    mx.array = np.asarray
    for name in ("uint8", "uint16", "uint32", "bfloat16", "float32", "int32"):
        setattr(mx, name, name)
    mx.fast = types.SimpleNamespace()
    pkg = types.ModuleType("mlx")
    pkg.core = mx
    sys.modules["mlx"], sys.modules["mlx.core"] = pkg, mx


def bf16_words(a: np.ndarray) -> np.ndarray:
    """float32 -> BF16 bit patterns, round to nearest even."""
    v = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    return ((v + 0x7FFF + ((v >> 16) & 1)) >> 16).astype(np.uint16)


def benchmark_tensor(rng, shape, zeros: bool):
    """N(0, 0.02) with 0.1 % of entries x64 and, optionally, 0.01 % set to +-0 or subnormals."""
    w = rng.standard_normal(shape).astype(np.float32) * 0.02
    w[rng.random(shape) < 1e-3] *= 64
    u = bf16_words(w)
    if zeros:
        hit = rng.random(shape) < 1e-2  # denser than the benchmark so a small tensor has some
        u[hit] = rng.choice(np.array([0x0000, 0x8000, 0x0001, 0x807F, 0x0040], np.uint16), size=int(hit.sum()))
    return u


def exponent_cases(rng):
    geo = lambda shape: np.clip(126 - rng.geometric(0.45, size=shape), 0, 255).astype(np.uint8)
    yield "geometric_20x1000", geo((20, 1000))
    yield "one_value_8x256", np.full((8, 256), 120, np.uint8)
    yield "all_values_4x512", np.tile(np.arange(256, dtype=np.uint8), (4, 2))
    spiky = geo((12, 512))
    spiky[:, 5::128] = 3
    yield "spike_per_tile_12x512", spiky
    yield "zero_or_255_16x384", np.where(rng.random((16, 384)) < 0.5, 0, 255).astype(np.uint8)
    yield "uniform_16x300", rng.integers(0, 256, size=(16, 300), dtype=np.uint8)
    yield "row_of_5", geo((1, 5))
    yield "single_weight", np.array([[77]], np.uint8)
    yield "short_rows_40x100", geo((40, 100))
    yield "experts_24x704", geo((24, 704))
    yield "k4_40x4", geo((40, 4))


def main(ref: Path):
    sys.path.insert(0, str(ref))
    _stub_mlx()
    from binade import bf16, rice
    from binade import format as fmt

    rng = np.random.default_rng(20240)
    out = {}
    for name, exps in exponent_cases(rng):
        table, rank = fmt.rank_table(np.bincount(exps.ravel(), minlength=256))
        enc = rice.encode(exps, table, rank)
        ranks, end = rice.decode_ranks(enc.meta, enc.bits, enc.roff, exps.shape[1])
        assert np.array_equal(rice.decode(enc, *exps.shape), exps)
        for k, v in (("exps", exps), ("table", table), ("rank", rank), ("meta", enc.meta), ("bits", enc.bits), ("roff", enc.roff), ("ranks", ranks.astype(np.uint8)), ("end", end)):
            out[f"{name}/{k}"] = v
    # the reference's hand-computed known-answer vector, re-derived by its own encoder
    meta, words, roff = rice.encode_ranks(np.array([[0, 1, 5, 2]]))
    out["by_hand/meta"], out["by_hand/bits"], out["by_hand/roff"] = meta, words, roff
    # rank ties and absent exponents
    hist = np.zeros(256, np.int64)
    hist[[3, 9, 120, 121, 200]] = [7, 7, 50, 7, 1]
    out["ties/hist"] = hist
    out["ties/table"], out["ties/rank"] = fmt.rank_table(hist)
    np.savez_compressed(HERE / "codec_cases.npz", **out)

    w = benchmark_tensor(rng, (96, 704), zeros=True)
    raw, exps = bf16.split(w)
    table, rank = fmt.rank_table(np.bincount(exps.ravel(), minlength=256))
    enc = rice.encode(exps, table, rank)
    assert np.array_equal(bf16.join(raw, rice.decode(enc, *w.shape)), w)
    np.savez_compressed(HERE / "config1_small.npz", w=w, raw=raw, exps=exps, table=table, rank=rank, meta=enc.meta, bits=enc.bits, roff=enc.roff)

    from binade.mlx.kernel import R4Matrix

    r4, f1 = {}, {}
    for name, shape in (("bench_16x512", (16, 512)), ("bench_8x128", (8, 128)), ("wide_6x1280", (6, 1280))):
        w = benchmark_tensor(rng, shape, zeros=False)
        w[::3, 7::61] = 0x7F80 - 0x0080 * rng.integers(1, 40, size=w[::3, 7::61].shape).astype(np.uint16)  # rare large exponents -> escapes
        raw, exps = bf16.split(w)
        table, rank = fmt.rank_table(np.bincount(exps.ravel(), minlength=256))
        e1 = fmt.encode(exps, table, rank)
        m = R4Matrix(raw, table, e1.meta, e1.idx, e1.esc)
        for k, v in (("w", w), ("raw", raw), ("table", table), ("rank", rank), ("codes", m.codes), ("flags", m.flags), ("esc", m.esc), ("row_esc", m.row_esc)):
            r4[f"{name}/{k}"] = np.asarray(v)
        for k, v in (("meta", e1.meta), ("idx", e1.idx), ("esc", e1.esc)):
            f1[f"{name}/{k}"] = v
        assert np.array_equal(fmt.decode(e1, *shape), exps)
    np.savez_compressed(HERE / "r4_layout.npz", **r4)
    np.savez_compressed(HERE / "format1.npz", **f1)

    # file level: a tiny model written with the reference's own streaming writer, packed by the
    # reference's packer; the packed shard is committed byte for byte
    from binade import st
    from binade.pack import pack_model
    from binade.unpack import PackedModel

    pm_dir = HERE / "packed_model"
    src, packed = pm_dir / "src", pm_dir / "packed"
    for d in (src, packed):
        d.mkdir(parents=True, exist_ok=True)
    tensors = {
        "model.embed_tokens.weight": benchmark_tensor(rng, (300, 256), zeros=True),
        "model.layers.0.self_attn.q_proj.weight": benchmark_tensor(rng, (260, 300), zeros=False),
        "model.layers.0.experts.gate_up_proj": benchmark_tensor(rng, (3, 256, 256), zeros=False),
        "model.layers.0.input_layernorm.weight": benchmark_tensor(rng, (256,), zeros=False),
        "lm_head.weight": benchmark_tensor(rng, (300, 256), zeros=False),
    }
    tensors["model.embed_tokens.weight"][3, :5] = [0x7FC0, 0x7F80, 0xFF80, 0x0000, 0x8000]  # NaN, +-Inf, +-0
    w = st.Writer(src / "model.safetensors", 4096)
    for name, u in tensors.items():
        w.add(name, u, "BF16")
    w.add("model.layers.0.linear_attn.A_log", rng.standard_normal(32).astype(np.float32))
    w.close()
    (src / "config.json").write_text(json.dumps({"model_type": "test", "hidden_size": 256}))
    pack_model(src, packed, chunk=5000, log=lambda *_: None, version="2")
    pm = PackedModel(packed, gpu=False)
    for name, u in tensors.items():
        assert np.array_equal(pm.tensor(name), u), name
    digest = hashlib.sha256((packed / "model.safetensors").read_bytes()).hexdigest()
    (pm_dir / "SHA256").write_text(f"{digest}  packed/model.safetensors\n")
    (packed / "binade_pack.json").unlink()  # holds wall time and a git commit: not reproducible
    print("golden vectors written;", digest)


if __name__ == "__main__":
    main(Path(sys.argv[1]))
