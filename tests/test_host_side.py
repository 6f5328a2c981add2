"""Host-side package code (no GPU): encoder, rank table, safetensors I/O, packer, classifier,
and the C-ABI libraries' exported symbols."""

import ctypes
import hashlib
import json
import re
from pathlib import Path

import numpy as np
import pytest

from binade_b200 import _native, bf16, classify, pack, rice, st
from binade_b200.format import TILE, rank_table
from conftest import GOLDEN, ROOT, golden
from oracle import oracle as o

CODEC = golden("codec_cases.npz")
CASES = [c for c in CODEC if "exps" in CODEC[c]]


def test_abi_exports_every_declared_symbol():
    """Every function declared in include/binade_b200.h is exported by one of the two libraries."""
    header = (ROOT / "include" / "binade_b200.h").read_text()
    declared = set(re.findall(r"\b(bn_\w+)\s*\(", header)) - {"bn_r4"}
    assert len(declared) >= 14
    exported = set()
    for which in ("cuda", "host"):
        lib = _native.load(which)
        for name in _native.symbols(which):
            assert hasattr(lib, name), name
            exported.add(name)
    assert declared == exported
    assert _native.load("cuda").bn_abi_version() == 201


def test_bad_arguments_are_refused_without_a_gpu():
    lib = _native.load("cuda")
    assert lib.bn_rice_ranks(None, None, 0, None, 4, 128, None, None, None) == 1
    assert b"null" in lib.bn_last_error()
    with pytest.raises(_native.NativeError):
        _native.call("host", "bn_host_rank_table", None, None, None)


def test_bf16_split_join_every_pattern():
    w = np.arange(1 << 16, dtype=np.uint32).astype(np.uint16)
    r, e = bf16.split(w)
    assert r.dtype == np.uint8 and e.dtype == np.uint8
    assert np.array_equal(bf16.join(r, e), w)
    ro, eo = o.np_split(w)
    assert np.array_equal(r, ro) and np.array_equal(e, eo)
    import torch

    t = torch.from_numpy(w.view(np.int16))
    rt, et = bf16.split(t)
    assert np.array_equal(rt.numpy(), r) and np.array_equal(et.numpy(), e)
    assert np.array_equal(bf16.join(rt, et).view(torch.int16).numpy().view(np.uint16), w)


@pytest.mark.parametrize("case", CASES)
def test_encoder_matches_reference_vectors(case):
    g = CODEC[case]
    table, rank = rank_table(np.bincount(g["exps"].ravel(), minlength=256))
    assert np.array_equal(table, g["table"]) and np.array_equal(rank, g["rank"])
    enc = rice.encode(g["exps"], table, rank)
    assert np.array_equal(enc.meta, g["meta"]) and np.array_equal(enc.bits, g["bits"]) and np.array_equal(enc.roff, g["roff"])
    assert enc.meta.size == g["exps"].shape[0] * -(-g["exps"].shape[1] // TILE)
    assert enc.nbits() == 8 * 256 + 8 * enc.meta.size + 32 * enc.bits.size + 32 * enc.roff.size


def test_encoder_hand_computed_stream():
    meta, words, roff = rice.encode_ranks(np.array([[0, 1, 5, 2]]))
    stream = [0, 1, 1, 0, 0, 0, 1, 1, 1, 0]
    assert meta.tolist() == [1 | 2 << 2] and roff.tolist() == [0]
    assert words.tolist() == [sum(b << i for i, b in enumerate(stream))]


def test_encoder_threads_and_chunks_agree():
    """Any thread count gives the same stream; row chunks encoded apart join by shifting roff."""
    rng = np.random.default_rng(4)
    ranks = np.minimum(rng.geometric(0.4, size=(30, 520)) - 1, 255).astype(np.uint8)
    one = rice.encode_ranks(ranks, threads=1)
    for t in (2, 7, 0):
        for a, b in zip(one, rice.encode_ranks(ranks, threads=t)):
            assert np.array_equal(a, b)
    parts = [rice.encode_ranks(ranks[a:b]) for a, b in ((0, 7), (7, 8), (8, 30))]
    base = np.cumsum([0] + [p[1].size for p in parts[:-1]])
    assert np.array_equal(np.concatenate([p[0] for p in parts]), one[0])
    assert np.array_equal(np.concatenate([p[1] for p in parts]), one[1])
    assert np.array_equal(np.concatenate([p[2] + np.uint32(b) for p, b in zip(parts, base)]), one[2])
    back, _ = o.c_rice_decode_ranks(*one, 520)
    assert np.array_equal(back, ranks)


def test_encoder_limits():
    meta, _, _ = rice.encode_ranks(np.full((1, TILE), 255))
    assert (meta[0] & 3) >= 2 and (meta[0] >> 2) == 255 >> (meta[0] & 3)
    with pytest.raises(ValueError):
        rice.encode_ranks(np.full((1, 4), 256))
    assert rice.encode_ranks(np.zeros((0, 8), np.uint8))[1].size == 0


def test_pack_tensor_level_matches_oracle():
    g = golden("config1_small.npz")[""]
    p = pack.pack(g["w"])
    for k in ("raw", "table", "meta", "bits", "roff"):
        assert np.array_equal(p[k], g[k]), k
    assert 10.0 < pack.bits_per_weight(p) < 12.0


def _source_model(tmp_path) -> Path:
    """Rebuild the golden source model from the committed source shard."""
    src = tmp_path / "src"
    src.mkdir()
    for f in (GOLDEN / "packed_model" / "src").iterdir():
        (src / f.name).write_bytes(f.read_bytes())
    return src


def test_pack_model_is_byte_identical_to_the_reference(tmp_path):
    src, out = _source_model(tmp_path), tmp_path / "packed"
    report = pack.pack_model(src, out, chunk=5000, log=lambda *_: None, version="2")
    want = GOLDEN / "packed_model" / "packed"
    got = (out / "model.safetensors").read_bytes()
    assert got == (want / "model.safetensors").read_bytes()
    assert hashlib.sha256(got).hexdigest() == (GOLDEN / "packed_model" / "SHA256").read_text().split()[0]
    assert (out / st.INDEX).read_text() == (want / st.INDEX).read_text()
    assert (out / "config.json").read_text() == (want / "config.json").read_text()
    assert pack.pack_meta(out) == pack.quant("2") and pack.pack_meta(src) is None
    assert report["packed_bits"] < 16 * report["packed_numel"]
    infos = {i.name: i for i in st.list_tensors(out)}
    assert "model.layers.0.input_layernorm.weight" in infos and "lm_head.weight.bits" in infos
    with pytest.raises(ValueError):
        pack.pack_model(src, tmp_path / "x", version="3")


def test_pack_model_format1_is_byte_identical_to_the_reference(tmp_path):
    """pack_model(version="1"): the shard the reference's packer wrote for the same source model
    (tests/golden/make_golden_format1_model.py), byte for byte, index included."""
    src, out = _source_model(tmp_path), tmp_path / "packed1"
    report = pack.pack_model(src, out, chunk=5000, log=lambda *_: None, version="1")
    want = GOLDEN / "packed_model" / "packed_v1"
    got = (out / "model.safetensors").read_bytes()
    assert got == (want / "model.safetensors").read_bytes()
    assert hashlib.sha256(got).hexdigest() == (GOLDEN / "packed_model" / "SHA256_v1").read_text().split()[0]
    assert (out / st.INDEX).read_text() == (want / st.INDEX).read_text()
    assert pack.pack_meta(out) == pack.quant("1")
    infos = {i.name: i for i in st.list_tensors(out)}
    assert "lm_head.weight.idx" in infos and "lm_head.weight.esc" in infos and "lm_head.weight.bits" not in infos
    assert report["packed_bits"] < 16 * report["packed_numel"]
    with pytest.raises(ValueError):
        pack.pack_model(src, tmp_path / "y", version="1", gpu=True)


@pytest.mark.parametrize("shape", [(16, 512), (8, 128), (6, 1280), (5, 100), (3, 1), (40, 4), (2, 2000)])
def test_format1_encoder_matches_the_restated_reference(shape):
    """format.encode_words (C++, all cores) against the numpy restatement of binade/format.py on
    short last tiles, rows shorter than a tile, rare large exponents (escape mode) and uniformly
    random words (fixed widths up to 8 bits)."""
    from binade_b200 import format as fmt

    rng = np.random.default_rng(sum(shape))
    for kind in ("normal", "uniform", "const"):
        if kind == "normal":
            w = (rng.standard_normal(shape) * 0.02).astype(np.float32)
            u = (w.view(np.uint32) >> 16).astype(np.uint16)
            u.reshape(-1)[3::17] = 0x7F80 - 0x0080 * rng.integers(1, 40, size=u.reshape(-1)[3::17].shape).astype(np.uint16)
        elif kind == "uniform":
            u = rng.integers(0, 1 << 16, size=shape, dtype=np.uint16)
        else:
            u = np.full(shape, 0x3C00, np.uint16)
        exps = ((u >> 7) & 0xFF).astype(np.uint8)
        table, rank = fmt.rank_table(np.bincount(exps.ravel(), minlength=256))
        meta, idx, esc = fmt.encode_words(u, rank)
        want_meta, want_idx, want_esc = o.np_f1_encode(exps, table, rank)
        assert np.array_equal(meta, want_meta) and np.array_equal(idx, want_idx) and np.array_equal(esc, want_esc), kind
        assert np.array_equal(o.np_f1_decode(meta, idx, esc, table, *shape), exps)


def test_format1_encoder_golden():
    """The reference's own format-1 arrays (tests/golden/format1.npz, written by its encoder)."""
    from binade_b200 import format as fmt

    f1, r4 = golden("format1.npz"), golden("r4_layout.npz")
    assert len(f1) >= 3
    for case in f1:
        meta, idx, esc = fmt.encode_words(r4[case]["w"], r4[case]["rank"])
        assert np.array_equal(meta, f1[case]["meta"]) and np.array_equal(idx, f1[case]["idx"]) and np.array_equal(esc, f1[case]["esc"]), case


def test_st_reader_and_writer(tmp_path):
    rng = np.random.default_rng(1)
    a = rng.integers(0, 1 << 16, size=(6, 10), dtype=np.uint16)
    b = rng.standard_normal(5).astype(np.float32)
    w = st.Writer(tmp_path / "model.safetensors", 1000, {"k": "v"})
    w.add("a.weight", a, "BF16")
    w.begin("b", "F32", b.shape)
    w.write(b[:2])
    w.write(b[2:])
    w.end()
    w.close()
    header, start = st.read_header(tmp_path / "model.safetensors")
    assert header["__metadata__"] == {"k": "v"} and start == 8 + 1000
    infos = {i.name: i for i in st.list_tensors(tmp_path)}
    assert infos["a.weight"].dtype == "BF16" and infos["a.weight"].rows == 6
    assert np.array_equal(st.read(infos["a.weight"]), a)
    assert np.array_equal(st.read(infos["a.weight"], (2, 5)), a[2:5])
    assert np.array_equal(st.read(infos["b"]), b)
    from safetensors import safe_open

    with safe_open(str(tmp_path / "model.safetensors"), framework="numpy") as f:
        assert set(f.keys()) == {"a.weight", "b"} and np.array_equal(f.get_tensor("b"), b)
    bad = st.Writer(tmp_path / "bad.safetensors", 8)
    bad.add("x" * 50, a)
    with pytest.raises(ValueError):
        bad.close()
    w2 = st.Writer(tmp_path / "short.safetensors", 512)
    w2.begin("t", "U8", (4,))
    w2.write(np.zeros(3, np.uint8))
    with pytest.raises(ValueError):
        w2.end()
    with pytest.raises(FileNotFoundError):
        st.shard_files(tmp_path / "nothing_here")


@pytest.mark.parametrize(
    "name,shape,dtype,cls,sub",
    [
        ("model.layers.3.self_attn.q_proj.weight", (4096, 3840), "BF16", "linear", "attn"),
        ("model.layers.3.mlp.down_proj.weight", (3840, 15360), "BF16", "linear", "mlp"),
        ("model.layers.0.experts.gate_up_proj", (128, 1408, 2816), "BF16", "linear", "experts"),
        ("model.layers.1.linear_attn.in_proj.weight", (512, 512), "BF16", "linear", "linattn"),
        ("model.embed_tokens.weight", (1000, 256), "BF16", "embed", "embed_tokens"),
        ("lm_head.weight", (1000, 256), "BF16", "embed", "lm_head"),
        ("model.embed_tokens_per_layer.weight", (1000, 256), "BF16", "ple", "ple"),
        ("model.vision_tower.blocks.0.attn.q_proj.weight", (512, 512), "BF16", "mm", "mm"),
        ("model.layers.0.input_layernorm.weight", (256,), "BF16", "other", "norm"),
        ("model.layers.0.mlp.router.weight", (128, 2816), "BF16", "other", "other"),
        ("model.layers.0.self_attn.q_proj.weight", (128, 128), "BF16", "other", "other"),
        ("model.layers.0.self_attn.q_proj.weight", (512, 512), "F32", "other", "other"),
    ],
)
def test_classify(name, shape, dtype, cls, sub):
    k = classify.classify(name, shape, dtype)
    assert (k.cls, k.sub) == (cls, sub)


def test_classify_layer_and_packable():
    k = classify.classify("model.layers.12.mlp.up_proj.weight", (512, 512), "BF16")
    assert k.layer == 12 and k.block == "model.layers.12"
    assert classify.classify("mtp.layers.0.mlp.up_proj.weight", (512, 512), "BF16").layer is None
    info = st.TensorInfo("model.vision_tower.conv.weight", "BF16", (1024, 1, 5), Path("x"), 0, 0)
    assert not pack.packable(info, pack.CLASSES)
    info = st.TensorInfo("lm_head.weight", "BF16", (300, 256), Path("x"), 0, 0)
    assert pack.packable(info, pack.CLASSES) and not pack.packable(info, ("linear",))
    assert pack.spans(st.TensorInfo("t", "BF16", (10, 300), Path("x"), 0, 0), 1000) == [(0, 3), (3, 6), (6, 9), (9, 10)]


def test_gpu_only_paths_fail_loudly_without_a_device():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a device is present")
    from binade_b200 import unpack

    g = golden("config1_small.npz")[""]
    with pytest.raises(RuntimeError, match="CUDA"):
        unpack.unpack({k: g[k] for k in ("raw", "table", "meta", "bits", "roff")})
    with pytest.raises(NotImplementedError):
        unpack.PackedModel(GOLDEN / "packed_model" / "packed", gpu=False)


def test_cli_pack_writes_both_formats(tmp_path):
    """`python -m binade_b200.cli pack SRC --out DIR [--format 1]`: the command line reaches the
    packer with its options, and the shards are the golden ones."""
    import subprocess
    import sys

    src = _source_model(tmp_path)
    for version, want in (("2", "packed"), ("1", "packed_v1")):
        out = tmp_path / f"cli{version}"
        r = subprocess.run([sys.executable, "-m", "binade_b200.cli", "pack", str(src), "--out", str(out), "--format", version], cwd=ROOT, capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
        assert "bits/weight" in r.stdout
        assert (out / "model.safetensors").read_bytes() == (GOLDEN / "packed_model" / want / "model.safetensors").read_bytes()
    bad = subprocess.run([sys.executable, "-m", "binade_b200.cli", "frobnicate"], cwd=ROOT, capture_output=True, text=True)
    assert bad.returncode != 0 and "usage" in (bad.stderr + bad.stdout)
