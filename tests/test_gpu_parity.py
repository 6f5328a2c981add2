"""GPU parity: every CUDA entry point, called through the C ABI, against the CPU oracle.

Bit-exact for the integer work (Rice decode, R4 expansion, dense decode); the fused products are
compared bit for bit with the oracle's same-order fp32 sums and with a PyTorch fp32 reference
that adds in the same order."""

import numpy as np
import pytest
import torch

from conftest import GOLDEN, golden
from oracle import oracle as o

pytestmark = pytest.mark.gpu

CODEC = golden("codec_cases.npz")
CASES = [c for c in CODEC if "exps" in CODEC[c]]


def bf16_words(a: np.ndarray) -> np.ndarray:
    v = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    return ((v + 0x7FFF + ((v >> 16) & 1)) >> 16).astype(np.uint16)


def weights(rng, shape, scale=0.02, escapes=True):
    """BF16 words: row-scaled normal values, some -0, a few rare large exponents (escapes)."""
    w = rng.standard_normal(shape) * scale * np.exp(rng.standard_normal(shape[:-1] + (1,)))
    u = bf16_words(w)
    flat = u.reshape(-1)
    flat[::997] = 0x8000
    if escapes:
        flat[5::199] = 0x3F80 | 0x4000
        flat[11::311] = bf16_words(np.array([3.0e-9], np.float32))[0]
    return u


def words(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def dev(a: np.ndarray) -> torch.Tensor:
    from binade_b200.cuda import kernels as ck

    return ck.to_device(a)


def packed_arrays(u: np.ndarray) -> dict:
    from binade_b200 import pack

    return pack.pack(u)


def torch_same_order(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """PyTorch fp32 reference of the documented order: x [M,K], w [N,K] bfloat16 -> [M,N] bfloat16.
    Lane l owns columns 128t + 4l + j; per lane sequential fp32 adds over t then j; lanes combine
    with strides 16, 8, 4, 2, 1; one rounding to BF16."""
    M, K = x.shape
    N = w.shape[0]
    T = -(-K // 128)
    xf = torch.zeros((M, T * 128), dtype=torch.float32, device=x.device)
    wf = torch.zeros((N, T * 128), dtype=torch.float32, device=x.device)
    xf[:, :K], wf[:, :K] = x.float(), w.float()
    real = (torch.arange(T * 128, device=x.device) < K).view(T, 32, 4)
    xf, wf = xf.view(M, 1, T, 32, 4), wf.view(1, N, T, 32, 4)
    acc = torch.zeros((M, N, 32), dtype=torch.float32, device=x.device)
    for t in range(T):
        for j in range(4):
            prod = wf[:, :, t, :, j] * xf[:, :, t, :, j]  # exact: two BF16 factors
            acc = torch.where(real[t, :, j], acc + prod, acc)
    for s in (16, 8, 4, 2, 1):
        acc = acc[..., :s] + acc[..., s : 2 * s]
    return acc[..., 0].to(torch.bfloat16)


# ------------------------------------------------------------------------------ Rice encode on the GPU
@pytest.mark.parametrize("shape,kind", [((64, 704), "normal"), ((160, 2112), "normal"), ((300, 260), "normal"), ((48, 100), "normal"), ((40, 4), "normal"), ((7, 1), "normal"), ((17, 15360), "normal"), ((5, 2, 384), "normal"), ((64, 1024), "uniform"), ((3, 16384), "uniform"), ((33, 130), "all_patterns"), ((20, 512), "const"), ((9, 257), "one_outlier")])
def test_rice_encode_on_gpu_matches_host(shape, kind):
    """bn_bf16_split_hist / bn_rice_encode_plan / bn_rice_encode_write against the host encoder
    (itself pinned to the reference's streams): every file array byte for byte, for short last
    tiles, K < 4, K not a multiple of 4, 3-D tensors, uniformly random words (large qmax, every
    k), every BF16 pattern, a constant tensor (no unary plane) and a lone outlier per tile (the
    longest unary runs); and the decoder gives the words back."""
    from binade_b200 import pack, unpack
    from binade_b200.cuda import kernels as ck

    rng = np.random.default_rng(sum(shape))
    if kind == "normal":
        u = weights(rng, shape)
    elif kind == "uniform":
        u = rng.integers(0, 1 << 16, size=shape, dtype=np.uint16)
    elif kind == "all_patterns":
        u = np.resize(np.arange(1 << 16, dtype=np.uint16), shape)
    elif kind == "const":
        u = np.full(shape, 0x3C00, np.uint16)
    else:
        u = np.full(shape, 0x3C00, np.uint16)
        u[:, ::97] = 0x7F7F
        u[:, 5::89] = 0x0001
    want = pack.pack(u)
    got = ck.rice_encode(ck.to_device(u.view(np.int16)))
    assert got["shape"] == want["shape"]
    for key, dt in (("raw", np.uint8), ("table", np.uint8), ("meta", np.uint8), ("bits", np.uint32), ("roff", np.uint32)):
        a = got[key].cpu().numpy()
        a = a.view(dt) if a.dtype.itemsize == np.dtype(dt).itemsize else a
        assert np.array_equal(a.reshape(want[key].shape), want[key]), key
    via_numpy = pack.pack(u, gpu=True)
    assert all(np.array_equal(via_numpy[key], want[key]) for key in ("raw", "table", "meta", "bits", "roff"))
    assert np.array_equal(unpack.unpack(via_numpy), u)


def test_pack_model_on_gpu_is_byte_identical_to_the_reference(tmp_path):
    """pack_model(gpu=True): the packed shard is the file the reference's packer wrote (the same
    golden file the host path is held to), chunked so that a tensor is encoded in several spans."""
    from binade_b200 import pack

    src = tmp_path / "src"
    src.mkdir()
    for f in (GOLDEN / "packed_model" / "src").iterdir():
        (src / f.name).write_bytes(f.read_bytes())
    out = tmp_path / "packed"
    pack.pack_model(src, out, chunk=5000, log=lambda *_: None, version="2", gpu=True)
    want = GOLDEN / "packed_model" / "packed" / "model.safetensors"
    assert (out / "model.safetensors").read_bytes() == want.read_bytes()


@pytest.mark.parametrize("case", CASES)
def test_rice_encode_on_gpu_golden(case):
    """The reference's own streams (golden cases written by its encoder) from the GPU encoder."""
    from binade_b200.cuda import kernels as ck

    g = CODEC[case]
    exps = g["exps"].astype(np.uint16)
    u = (exps << 7).astype(np.uint16)  # words whose exponent bytes are the case's
    got = ck.rice_encode(ck.to_device(u.view(np.int16)))
    if "table" in g:
        assert np.array_equal(got["table"].cpu().numpy(), g["table"])
    assert np.array_equal(got["meta"].cpu().numpy(), g["meta"])
    assert np.array_equal(got["bits"].cpu().numpy().view(np.uint32), g["bits"])
    assert np.array_equal(got["roff"].cpu().numpy().view(np.uint32), g["roff"])


# ------------------------------------------------------------------------------ Rice decode
@pytest.mark.parametrize("case", CASES)
def test_rice_ranks_golden(case):
    from binade_b200.cuda import kernels as ck

    g = CODEC[case]
    R, K = g["exps"].shape
    ranks, rend = ck.rice_ranks(dev(g["meta"]), dev(g["bits"]), dev(g["roff"]), K)
    got = ranks.cpu().numpy()
    assert np.array_equal(got[:, :K], g["ranks"])
    assert not got[:, K:].any()
    assert np.array_equal(rend.cpu().numpy().view(np.uint32), (g["end"] + 31) >> 5)


@pytest.mark.parametrize("R,K", [(1, 5), (40, 100), (24, 704), (64, 1000), (7, 256), (300, 3840), (33, 15360)])
def test_rice_ranks_shapes(R, K):
    from binade_b200 import rice
    from binade_b200.cuda import kernels as ck

    rng = np.random.default_rng(K)
    ranks = np.minimum(rng.geometric(0.35, size=(R, K)) - 1, 255).astype(np.uint8)
    ranks[::5, ::97] = rng.integers(0, 256, size=ranks[::5, ::97].shape)
    meta, bits, roff = rice.encode_ranks(ranks)
    ref, end = o.c_rice_decode_ranks(meta, bits, roff, K)
    assert np.array_equal(ref, ranks)
    got, rend = ck.rice_ranks(dev(meta), dev(bits), dev(roff), K)
    got, rend = got.cpu().numpy(), rend.cpu().numpy().view(np.uint32)
    assert np.array_equal(got[:, :K], ranks) and not got[:, K:].any()
    assert np.array_equal(rend, (end + 31) >> 5)
    assert np.array_equal(rend, np.append(roff[1:], bits.size))


def test_rice_decode_and_errors():
    from binade_b200 import rice

    g = CODEC["geometric_20x1000"]
    enc = rice.RiceEncoded(g["table"], g["meta"], g["bits"], g["roff"])
    assert np.array_equal(rice.decode(enc, 20, 1000), g["exps"])
    with pytest.raises(ValueError):
        rice.decode(rice.RiceEncoded(g["table"], g["meta"], g["bits"][:-1], g["roff"]), 20, 1000)
    with pytest.raises(ValueError):
        rice.decode(enc, 19, 1000)


def test_every_bf16_pattern_round_trips():
    from binade_b200 import pack, unpack

    w = np.random.default_rng(1).permutation(np.arange(1 << 16, dtype=np.uint32).astype(np.uint16)).reshape(256, 256)
    assert np.array_equal(unpack.unpack(pack.pack(w)), w)


@pytest.mark.parametrize("shape", [(96, 704), (7, 5), (3, 40, 100), (1, 1)])
def test_pack_unpack_round_trip(shape):
    from binade_b200 import pack, unpack

    u = weights(np.random.default_rng(sum(shape)), shape)
    p = pack.pack(u)
    assert np.array_equal(unpack.unpack(p), u)
    if u.size > 4:
        bad = dict(p, bits=p["bits"][:-1])
        with pytest.raises(ValueError):
            unpack.unpack(bad)


def test_packed_model_restores_every_tensor(tmp_path):
    from binade_b200 import st
    from binade_b200.unpack import PackedModel

    pm = PackedModel(GOLDEN / "packed_model" / "packed")
    orig = {i.name: i for i in st.list_tensors(GOLDEN / "packed_model" / "src")}
    assert sorted(pm.names()) == sorted(orig)
    assert set(pm.packed) == {"model.embed_tokens.weight", "model.layers.0.self_attn.q_proj.weight", "model.layers.0.experts.gate_up_proj", "lm_head.weight"}
    for name, info in orig.items():
        assert np.array_equal(pm.tensor(name), st.read(info)), name
    rows = list(pm.rows("lm_head.weight", chunk=5000))
    assert len(rows) > 1 and rows[0][0] == 0 and rows[-1][1] == 300


# ------------------------------------------------------------------------------ Rice -> R4
@pytest.mark.parametrize("case", list(golden("r4_layout.npz")))
def test_transcode_golden_layout(case):
    from binade_b200.cuda import r4

    g = golden("r4_layout.npz")[case]
    a = r4.transcode(packed_arrays(g["w"]))
    assert np.array_equal(a["codes"].cpu().numpy().view(np.uint16), g["codes"])
    assert np.array_equal(a["flags"].cpu().numpy(), g["flags"])
    assert np.array_equal(a["esc"].cpu().numpy(), g["esc"])
    assert np.array_equal(a["row_esc"].cpu().numpy().view(np.uint32), g["row_esc"])
    assert np.array_equal(words(r4.R4Linear(a).dense()), g["w"])


@pytest.mark.parametrize("N,K", [(64, 704), (160, 2112), (300, 260), (48, 100), (64, 128), (40, 4), (300, 3840), (17, 15360)])
def test_transcode_matches_oracle(N, K):
    from binade_b200.cuda import r4

    u = weights(np.random.default_rng(K), (N, K))
    want = o.pack_r4(u)
    a = r4.transcode(packed_arrays(u))
    for k, dt in (("codes", np.uint16), ("flags", np.uint8), ("esc", np.uint8), ("row_esc", np.uint32)):
        got = a[k].cpu().numpy()
        assert np.array_equal(got.view(dt) if got.dtype.itemsize == np.dtype(dt).itemsize else got, want[k]), k
    assert np.array_equal(words(r4.R4Linear(a).dense()), u)
    assert a["shape"] == (N, K) and r4.r4_bytes(a) == sum(want[k].nbytes for k in ("raw", "codes", "flags", "esc", "table", "row_esc"))


@pytest.mark.parametrize("N,K,kind", [(7201, 260, "normal"), (3601, 132, "normal"), (7107, 4, "normal"), (3553, 3840, "normal"), (7300, 512, "uniform"), (3700, 384, "uniform"), (7200, 640, "mixed"), (3602, 1000, "mixed"), (7110, 128, "const")])
def test_transcode_many_rows(N, K, kind):
    """Row counts at which the expander runs four (N >= 7104) or two (N >= 3552) rows a warp:
    the arrays against the oracle, for short last tiles, a row count that leaves the last warp
    partly empty, uniformly random words (nearly every weight escapes, every plane count up to the
    format's largest), a mix of both by row, and a constant tensor (no unary plane at all)."""
    from binade_b200.cuda import r4

    rng = np.random.default_rng(N + K)
    if kind == "normal":
        u = weights(rng, (N, K))
    elif kind == "uniform":
        u = rng.integers(0, 1 << 16, size=(N, K), dtype=np.uint16)
    elif kind == "mixed":
        u = weights(rng, (N, K))
        rows = rng.random(N) < 0.3
        u[rows] = rng.integers(0, 1 << 16, size=(int(rows.sum()), K), dtype=np.uint16)
    else:
        u = np.full((N, K), 0x3C00, np.uint16)
    want = o.pack_r4(u)
    a = r4.transcode(packed_arrays(u))
    for k, dt in (("codes", np.uint16), ("flags", np.uint8), ("esc", np.uint8), ("row_esc", np.uint32)):
        got = a[k].cpu().numpy()
        assert np.array_equal(got.view(dt) if got.dtype.itemsize == np.dtype(dt).itemsize else got, want[k]), k
    assert np.array_equal(words(r4.R4Linear(a).dense()), u)


def test_transcode_all_escapes_grows_scratch():
    """Uniform exponents: nearly every weight escapes, far beyond the default scratch size."""
    from binade_b200.cuda import r4

    rng = np.random.default_rng(3)
    u = rng.integers(0, 1 << 16, size=(64, 1024), dtype=np.uint16)
    want = o.pack_r4(u)
    a = r4.transcode(packed_arrays(u))
    assert a["esc"].numel() - 1 > 64 * 1024 * 0.8
    assert np.array_equal(a["esc"].cpu().numpy(), want["esc"])
    assert np.array_equal(a["row_esc"].cpu().numpy().view(np.uint32), want["row_esc"])
    assert np.array_equal(words(r4.R4Linear(a).dense()), u)


@pytest.mark.parametrize("which", ["packed", "packed_v1"])
def test_streamed_load_equals_plain_load(which):
    """stream_r4 (reader thread -> pinned buffers -> copy stream -> expander) gives the arrays
    that reading every file array and transcoding it gives, for every packed weight of the golden
    packed models (format 2 and format 1, both written by the reference's packer), in the order
    asked for; the unpacked tensors are the source model's; a name that is not packed raises."""
    from binade_b200 import st
    from binade_b200.cuda import r4
    from binade_b200.cuda.stream_load import stream_r4
    from binade_b200.unpack import PackedModel

    pm = PackedModel(GOLDEN / "packed_model" / which)
    source = {i.name: i for i in st.list_tensors(GOLDEN / "packed_model" / "src")}
    for name in pm.packed:
        assert np.array_equal(pm.tensor(name), st.read(source[name])), name
    plain = {name: r4.transcode(h) for name, h in r4.holders(pm).items()}
    assert len(plain) >= 3
    seen = []
    for name, a in stream_r4(pm, slots=2):
        seen.append(name)
        for key in ("raw", "codes", "flags", "esc", "table", "row_esc"):
            assert torch.equal(a[key].reshape(-1), plain[name][key].reshape(-1)), (name, key)
        assert a["shape"] == plain[name]["shape"]
    assert seen == list(pm.packed)
    back = list(pm.packed)[::-1]
    assert [n for n, _ in stream_r4(pm, names=back, slots=1)] == back
    with pytest.raises(KeyError):
        list(stream_r4(pm, names=["no.such.weight"]))


def test_transcode_rejects_bad_input():
    from binade_b200.cuda import r4

    u = weights(np.random.default_rng(0), (8, 256))
    p = packed_arrays(u)
    with pytest.raises(ValueError):
        r4.transcode(dict(p, bits=p["bits"][:-1]))
    with pytest.raises(ValueError):
        r4.transcode(packed_arrays(weights(np.random.default_rng(0), (8, 6))))
    with pytest.raises(ValueError):
        r4.transcode(dict(p, roff=p["roff"][:-1]))


def test_dense_row_remap():
    """dense(n, rs, r0): rows r0 .. r0+n-1 of every block of rs storage rows (expert halves)."""
    from binade_b200.cuda import r4

    E, n, K = 4, 24, 384
    u = weights(np.random.default_rng(9), (E, 2 * n, K))
    m = r4.R4Linear(r4.transcode(packed_arrays(u)))
    assert np.array_equal(words(m.dense(n, 2 * n, 0)).reshape(E, n, K), u[:, :n])
    assert np.array_equal(words(m.dense(n, 2 * n, n)).reshape(E, n, K), u[:, n:])
    assert np.array_equal(words(m.dense()), u)


# ------------------------------------------------------------------------------ format 1
@pytest.mark.parametrize("name", ["bench_16x512", "bench_8x128", "wide_6x1280"])
def test_format1_golden_to_r4_and_bf16(name):
    """The reference's own format-1 encode output (golden) expands on the GPU to the R4 arrays
    the reference builds from it (binade/mlx/kernel.py R4Matrix) and unpacks to the tensor."""
    from binade_b200.cuda import kernels as ck
    from binade_b200.cuda import r4

    f1, lay = golden("format1.npz")[name], golden("r4_layout.npz")[name]
    w = lay["w"]
    R, K = w.shape
    a = r4.transcode({"raw": lay["raw"], "table": lay["table"], "meta": f1["meta"], "idx": f1["idx"], "esc": f1["esc"]})
    for k in ("codes", "flags", "esc", "row_esc"):
        got = a[k].cpu().numpy().view(lay[k].dtype).reshape(-1)
        assert np.array_equal(got, lay[k].reshape(-1)), k
    f = ck.Format1(f1["meta"], f1["idx"], f1["esc"], lay["table"], R, K)
    assert np.array_equal(words(f.unpack(lay["raw"])), w)
    assert np.array_equal(f.ranks().cpu().numpy()[:, :K], lay["rank"][o.np_split(w)[1]])


@pytest.mark.parametrize("R,K", [(40, 100), (7, 4), (33, 704), (12, 3840), (64, 128)])
def test_format1_shapes_against_oracle(R, K):
    """Ragged rows, zero-width tiles (a constant tile), fixed and escape tiles, all decoded like
    the oracle's restatement of format.decode; R4 arrays equal those of the format-2 path."""
    from binade_b200 import bf16
    from binade_b200.cuda import kernels as ck
    from binade_b200.cuda import r4
    from binade_b200.format import rank_table

    rng = np.random.default_rng(R * 1000 + K)
    u = weights(rng, (R, K))
    u[R // 2] = 0x3C00  # a constant row: its tiles need 0 bits
    raw, exps = o.np_split(u)
    table, rank = rank_table(np.bincount(exps.reshape(-1), minlength=256))
    meta, idx, esc = o.np_f1_encode(exps, table, rank)
    assert np.array_equal(o.np_f1_decode(meta, idx, esc, table, R, K), exps)
    f = ck.Format1(meta, idx, esc, table, R, K)
    assert np.array_equal(words(f.unpack(raw)), u)
    assert np.array_equal(f.ranks().cpu().numpy()[:, :K], rank[exps])
    if K % 4 == 0:
        a1 = r4.transcode({"raw": raw, "table": table, "meta": meta, "idx": idx, "esc": esc})
        a2 = r4.transcode(packed_arrays(u))
        for k in ("raw", "codes", "flags", "esc", "row_esc", "table"):
            assert torch.equal(a1[k].reshape(-1), a2[k].reshape(-1)), k
    with pytest.raises(ValueError):
        ck.Format1(meta, idx, esc[:-1] if esc.size else np.ones(1, np.uint8), table, R, K)
    with pytest.raises(ValueError):
        ck.Format1(meta, np.concatenate([idx, np.zeros(4, np.uint32)]), esc, table, R, K)


def test_format1_packed_file_unpacks_and_converts(tmp_path):
    """A packed shard in format 1 (name.raw/.table/.meta/.idx/.esc, as binade pack --format 1
    writes it): PackedModel restores the tensor and the hook runs on it."""
    from binade_b200 import st
    from binade_b200.cuda import r4
    from binade_b200.format import rank_table
    from binade_b200.unpack import PackedModel

    rng = np.random.default_rng(77)
    u = weights(rng, (3, 40, 256))
    raw, exps = o.np_split(u)
    table, rank = rank_table(np.bincount(exps.reshape(-1), minlength=256))
    meta, idx, esc = o.np_f1_encode(exps.reshape(-1, 256), table, rank)
    w = st.Writer(tmp_path / "model.safetensors", 4096)
    name = "model.layers.0.experts.down_proj"
    for suffix, arr in (("raw", raw), ("table", table), ("meta", meta), ("idx", idx), ("esc", esc)):
        w.add(f"{name}.{suffix}", arr)
    w.add("model.norm.weight", np.ones(8, np.float32))
    w.close()
    pm = PackedModel(tmp_path)
    assert pm.packed == [name] and np.array_equal(pm.tensor(name), u)
    assert len(list(pm.rows(name, chunk=256 * 16))) > 1
    h = r4.holders(pm)[name]
    m = r4.R4Linear(r4.transcode(h))
    assert np.array_equal(words(m.dense()), u)


# ------------------------------------------------------------------------------ embedding lookups
@pytest.mark.parametrize("N,K", [(1000, 384), (257, 100), (64, 4096), (33, 4)])
def test_embedding_lookups(N, K):
    """R4Embedding and RiceEmbedding return exactly the packed rows (reference r4.py:303-367), in
    any id order, with repeats; the oracle's decode of the same rows is the check."""
    from binade_b200.cuda import r4

    rng = np.random.default_rng(N + K)
    u = weights(rng, (N, K))
    p = packed_arrays(u)
    ranks, _ = o.c_rice_decode_ranks(p["meta"], p["bits"], p["roff"], K)
    want_all = o.np_join(np.asarray(p["raw"]).reshape(N, K), np.asarray(p["table"])[ranks[:, :K]])
    assert np.array_equal(want_all, u)
    ids = np.concatenate([rng.integers(0, N, 50), [0, N - 1, N - 1, 0]]).astype(np.int64).reshape(6, 9)
    e_r4 = r4.R4Embedding(r4.transcode(p))
    e_rice = r4.RiceEmbedding(p)
    for ids_t in (torch.from_numpy(ids).cuda(), torch.from_numpy(ids.astype(np.int32)).cuda(), torch.from_numpy(ids)):
        for e in (e_r4, e_rice):
            got = e(ids_t)
            assert got.shape == (6, 9, K) and got.dtype == torch.bfloat16
            assert np.array_equal(words(got), want_all[ids])
    assert np.array_equal(words(e_rice.dense()), u)
    assert np.array_equal(words(e_r4.dense()), u)
    # an id outside the table: a row of zeros, nothing read out of bounds
    bad = torch.tensor([N, 0, 2**31 - 1], dtype=torch.int64).cuda()
    for e in (e_r4, e_rice):
        got = words(e(bad))
        assert not got[0].any() and not got[2].any() and np.array_equal(got[1], u[0])
    assert e_r4(torch.zeros((0,), dtype=torch.int64)).shape == (0, K)


def test_convert_swaps_embedding_holders():
    from binade_b200.cuda import r4

    rng = np.random.default_rng(12)
    u1, u2 = weights(rng, (50, 128)), weights(rng, (40, 256))

    class Tiny(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.tok = r4.BinadeEmbedding(packed_arrays(u1))
            self.ple = r4.BinadeEmbedding(packed_arrays(u2), gather_only=True)

    m = Tiny()
    with pytest.raises(RuntimeError):
        m.tok(torch.zeros(1, dtype=torch.int64))
    assert r4.convert(m) == 2
    assert isinstance(m.tok, r4.R4Embedding) and isinstance(m.ple, r4.RiceEmbedding)
    ids = torch.tensor([[3, 49], [0, 3]]).cuda()
    assert np.array_equal(words(m.tok(ids)), u1[ids.cpu().numpy()])
    assert np.array_equal(words(m.ple(ids % 40)), u2[(ids % 40).cpu().numpy()])


def test_embedding_as_linear_is_the_matvec():
    from binade_b200.cuda import r4

    u = weights(np.random.default_rng(4), (96, 256))
    a = r4.transcode(packed_arrays(u))
    x = torch.randn(1, 256, device="cuda").to(torch.bfloat16)
    assert np.array_equal(words(r4.R4Embedding(a).as_linear(x)), words(r4.R4Linear(a)(x)))


# ------------------------------------------------------------------------------ fused products
@pytest.mark.parametrize("N,K", [(64, 704), (160, 2112), (300, 260), (48, 100), (64, 128), (40, 4), (4096, 512), (520, 3840), (200, 15360)])
def test_matvec_bit_exact(N, K):
    from binade_b200.cuda import r4

    rng = np.random.default_rng(N + K)
    u = weights(rng, (N, K))
    xw = bf16_words(rng.standard_normal((1, K)))
    m = r4.R4Linear(r4.transcode(packed_arrays(u)))
    x = dev(xw).view(torch.bfloat16)
    got = m(x)
    assert got.shape == (1, N) and got.dtype == torch.bfloat16
    want = o.c_r4_matvec(o.pack_r4(u), xw[0], N, K)
    assert np.array_equal(words(got)[0], want)
    ref = torch_same_order(x, dev(u).view(torch.bfloat16))
    assert np.array_equal(words(got), words(ref))


@pytest.mark.parametrize("N,K", [(7800, 640), (7701, 1296), (2100, 3840), (1925, 704), (600, 16384), (1500, 2816), (15360, 768)])
def test_matvec_rows_per_warp_shapes(N, K):
    """The batch-1 kernel walks four, two or one row per warp depending on the row count, with
    rings of different depths, full and short last tiles, one or several rounds per warp."""
    from binade_b200.cuda import r4

    rng = np.random.default_rng(N * 7 + K)
    u = weights(rng, (N, K))
    xw = bf16_words(rng.standard_normal((1, K)))
    m = r4.R4Linear(r4.transcode(packed_arrays(u)))
    got = m(dev(xw).view(torch.bfloat16))
    assert np.array_equal(words(got)[0], o.c_r4_matvec(o.pack_r4(u), xw[0], N, K))


@pytest.mark.parametrize("dense_escapes", [0.02, 0.5])
def test_matvec_rows_dense_with_escapes(dense_escapes):
    """Tiles with many escapes per thread and rows with more escapes than the register window
    holds: the general patch path and the window's refills."""
    from binade_b200.cuda import r4

    N, K = 2200, 1280
    rng = np.random.default_rng(17)
    u = weights(rng, (N, K))
    rare = bf16_words((2.0 ** np.arange(-60, 60, 1.5)).astype(np.float32))  # 80 exponents: most land past rank 14
    hit = rng.random((N, K)) < dense_escapes
    u[hit] = rare[rng.integers(0, len(rare), int(hit.sum()))]
    xw = bf16_words(rng.standard_normal((1, K)) * 1e-3)
    m = r4.R4Linear(r4.transcode(packed_arrays(u)))
    want = o.pack_r4(u)
    assert want["esc"].size - 1 > 0.5 * dense_escapes * N * K  # most of the rare exponents really escape
    got = m(dev(xw).view(torch.bfloat16))
    assert np.array_equal(words(got)[0], o.c_r4_matvec(want, xw[0], N, K))


@pytest.mark.parametrize("N,K,density", [(2200, 1280, 0.02), (2200, 1280, 0.5), (15392, 640, 0.003), (5000, 1200, 0.01), (300, 2064, 0.2), (37, 768, 0.05)])
def test_escape_columns_and_both_layouts(N, K, density):
    """bn_r4_esc_columns against its definition restated in numpy, and the one-row kernel with and
    without the derived arrays (a thread walking its own column of escapes, or the row's threads
    agreeing on positions): the same bits, for four and two rows a warp, short last tiles, rows
    with hundreds of escapes and several escapes in one code word."""
    from binade_b200.cuda import kernels as ck
    from binade_b200.cuda import r4

    rng = np.random.default_rng(N + K)
    u = weights(rng, (N, K))
    rare = bf16_words((2.0 ** np.arange(-60, 60, 1.5)).astype(np.float32))
    hit = rng.random((N, K)) < density
    u[hit] = rare[rng.integers(0, len(rare), int(hit.sum()))]
    a = r4.transcode(packed_arrays(u))
    plain = dict(a)  # the standard arrays only
    ck.r4_esc_columns(a)
    want = o.pack_r4(u)
    esc_cols, col_esc = o.esc_columns(want)
    n = want["esc"].size - 1
    assert n > 0.5 * density * N * K
    assert np.array_equal(a["esc_cols"].cpu().numpy(), esc_cols)
    assert np.array_equal(a["col_esc"].cpu().numpy().view(np.uint16), col_esc)
    xw = bf16_words(rng.standard_normal((1, K)) * 1e-3)
    x = dev(xw).view(torch.bfloat16)
    y = o.c_r4_matvec(want, xw[0], N, K)
    assert "esc_cols" not in plain
    assert np.array_equal(words(ck.r4_matvec(plain, x, N, K))[0], y)
    assert np.array_equal(words(ck.r4_matvec(a, x, N, K))[0], y)
    xm = dev(bf16_words(rng.standard_normal((16, K)) * 1e-3)).view(torch.bfloat16)  # the tensor-core kernel, both layouts
    assert np.array_equal(words(ck.r4_mma(plain, xm, N, K)), words(ck.r4_mma(a, xm, N, K)))


def test_linear_group_one_launch():
    """q, k, v (and gate, up) through bn_r4_rows_multi: the same bits as one call per matrix,
    for group sizes 1..4, unequal row counts, and a row count that is not a multiple of four."""
    from binade_b200.cuda import r4

    K = 1664
    rng = np.random.default_rng(3)
    Ns = [4096, 1022, 1024, 517]
    us = [weights(rng, (n, K)) for n in Ns]
    ms = [r4.R4Linear(r4.transcode(packed_arrays(u))) for u in us]
    xw = bf16_words(rng.standard_normal((1, K)))
    x = dev(xw).view(torch.bfloat16)
    for count in (1, 2, 3, 4):
        ys = r4.R4LinearGroup(ms[:count])(x)
        assert len(ys) == count
        for y, u, n in zip(ys, us, Ns):
            assert y.shape == (1, n)
            assert np.array_equal(words(y)[0], o.c_r4_matvec(o.pack_r4(u), xw[0], n, K))
    two_rows = torch.cat([x, x])
    for y, m in zip(r4.R4LinearGroup(ms[:2])(two_rows), ms):  # several rows: module by module
        assert np.array_equal(words(y), words(m(two_rows)))


def test_matvec_unaligned_input_falls_back():
    """An input vector that does not start on a 16-byte boundary (a view at an odd offset) is
    served by the plain-load kernel instead of the bulk-copy ones: same bits."""
    from binade_b200.cuda import kernels as ck
    from binade_b200.cuda import r4

    N, K = 700, 2048
    rng = np.random.default_rng(5)
    u = weights(rng, (N, K))
    xw = bf16_words(rng.standard_normal((1, K)))
    m = r4.R4Linear(r4.transcode(packed_arrays(u)))
    want = o.c_r4_matvec(o.pack_r4(u), xw[0], N, K)
    for shift in (1, 3, 4):
        buf = torch.zeros(K + 8, dtype=torch.bfloat16, device="cuda")
        buf[shift : shift + K] = dev(xw).view(torch.bfloat16)[0]
        x = buf[shift : shift + K]
        assert x.data_ptr() % 16 != 0
        assert np.array_equal(words(ck.r4_matvec(m._a, x, N, K)), want)
        xs = buf[shift : shift + K].reshape(1, K)
        assert np.array_equal(words(ck.r4_rows(m._a, xs, N, K))[0], want)


def adversarial(R: int, K: int, seed: int = 0) -> np.ndarray:
    """Rows whose sum with an all-ones input depends on the order: +2^25 first, then ones that
    vanish against it (fp32 ulp at 2^25 is 4), then -2^25: 0 in the documented order. Row types
    cycle: the pattern on one lane (columns 128j), on every 8th column, random values. The 2^25
    exponent is rare, so these rows also exercise escapes."""
    big = 2.0**25
    w = np.zeros((R, K), np.float32)
    last = 128 * ((K - 1) // 128)
    w[0::3, 0], w[0::3, last] = big, -big
    w[0::3, 128:last:128] = 1.0
    w[1::3, 0], w[1::3, K - 8] = big, -big
    w[1::3, 8 : K - 8 : 8] = 1.0
    w[2::3] = np.random.default_rng(seed).standard_normal(w[2::3].shape) * 0.02
    return bf16_words(w)


@pytest.mark.parametrize("N,K", [(96, 704), (4096, 512), (512, 2048), (48, 2816)])
def test_order_sensitive_rows(N, K):
    from binade_b200.cuda import r4

    u = adversarial(N, K)
    m = r4.R4Linear(r4.transcode(packed_arrays(u)))
    W = dev(u).view(torch.bfloat16)
    for M in (1, 2, 3, 8, 15, 16):
        x = torch.ones((M, K), dtype=torch.bfloat16, device="cuda")
        got = m.fused_rows(x)
        assert np.array_equal(words(got), words(torch_same_order(x, W))), M
        assert np.array_equal(words(got), o.c_dense_rows(words(x), u)), M
    y = words(m(torch.ones((1, K), dtype=torch.bfloat16, device="cuda")))[0]
    exact = o.bf16_to_f32(u).astype(np.float64).sum(axis=1)
    assert not y[0::3].any()  # lane pattern: exactly 0 in the documented order
    assert np.any(o.bf16_to_f32(y[1::3]) != exact[1::3])  # another grouping rounds differently


@pytest.mark.parametrize("M", [2, 4, 5, 8, 11, 16])
def test_small_m_rows(M):
    from binade_b200.cuda import r4

    N, K = 333, 1664
    rng = np.random.default_rng(M)
    u = weights(rng, (N, K))
    xw = bf16_words(rng.standard_normal((M, K)))
    m = r4.R4Linear(r4.transcode(packed_arrays(u)))
    got = m.fused_rows(dev(xw).view(torch.bfloat16).reshape(1, M, K))
    assert got.shape == (1, M, N)
    assert np.array_equal(words(got)[0], o.c_dense_rows(xw, u))


@pytest.mark.parametrize("M,N,K", [(16, 128, 128), (16, 256, 512), (32, 200, 3840), (128, 384, 1024), (24, 130, 264), (100, 96, 2048), (1, 64, 128), (256, 300, 768), (200, 1000, 1280), (300, 128, 256)])
def test_mma_rows_against_fp32(M, N, K):
    """Tensor-core decode GEMM: the weights it multiplies by are exactly the decoded BF16 weights
    (checked with one-hot inputs, where every output is a single weight), and on random inputs
    every output is within one BF16 unit in the last place of the fp32 product (plus the fp32
    summation noise of a differently ordered sum, 1e-5 of the output scale)."""
    from binade_b200.cuda import r4

    rng = np.random.default_rng(M * 7 + N + K)
    u = weights(rng, (N, K), escapes=False)
    u.reshape(-1)[3::173] = 0x5F80  # rare finite exponent: escapes
    m = r4.R4Linear(r4.transcode(packed_arrays(u)))
    w = dev(u).view(torch.bfloat16)
    # one-hot rows: output m is column k_m of W, exactly
    ks = rng.integers(0, K, M)
    x1 = torch.zeros((M, K), dtype=torch.bfloat16, device="cuda")
    x1[torch.arange(M), torch.from_numpy(ks).cuda()] = 1.0
    got1, want1 = words(m.mma_rows(x1)), u[:, ks].T.copy()
    want1[want1 == 0x8000] = 0  # a sum that starts at +0 turns a lone -0 product into +0
    assert np.array_equal(got1, want1)
    x = torch.randn((M, K), device="cuda").to(torch.bfloat16)
    got = m.mma_rows(x).float()
    ref = x.float() @ w.float().T
    scale = ref.abs().mean()
    bound = ref.abs() * 2.0**-7 + scale * 1e-5
    assert bool(((got - ref).abs() <= bound).all()), float(((got - ref).abs() - bound).max())


@pytest.mark.parametrize("N,K,density", [(333, 1040, 0.0), (1000, 1200, 0.002), (260, 2064, 0.1), (15392, 640, 0.001), (120, 128, 0.5)])
def test_mma_decodes_every_weight(N, K, density):
    """The tensor-core path with eight threads per weight row (K % 16 == 0, M <= 128): one-hot
    inputs over every column return every decoded weight exactly, with short last tiles, with
    rows dense in escapes (window slides, several escapes per thread) and with the largest block
    (104 rows on each of 148 SMs)."""
    from binade_b200.cuda import r4

    rng = np.random.default_rng(N + K)
    u = weights(rng, (N, K), escapes=False)
    if density:
        rare = (0x5F80 + 0x80 * np.arange(60)).astype(np.uint16)  # 60 large finite exponents (no Inf: 0 x Inf would turn whole outputs into NaN): most of them escape
        hit = rng.random(u.shape) < density
        u[hit] = rng.choice(rare, int(hit.sum()))
    m = r4.R4Linear(r4.transcode(packed_arrays(u)))
    if density:
        assert m._a["esc"].numel() - 1 > 0.5 * density * N * K
    for M in (128, 64, 16):  # three ring depths / stage counts
        for k0 in range(0, K, M):
            n = min(M, K - k0)
            x1 = torch.zeros((n, K), dtype=torch.bfloat16, device="cuda")
            x1[torch.arange(n), torch.arange(k0, k0 + n)] = 1.0
            want = u[:, k0 : k0 + n].T.copy()
            want[want == 0x8000] = 0  # a sum that starts at +0 turns a lone -0 product into +0
            assert np.array_equal(words(m.mma_rows(x1)), want), (M, k0)
            if N > 2000 and k0 >= 2 * M:
                break  # the big case: a few column blocks are enough


@pytest.mark.parametrize("N,K", [(384, 1024), (520, 3840), (256, 15360), (128, 16384)])
def test_mma_rows_in_the_order_of_cublas(N, K):
    """Split-K in the kernel (every slice from zero in its own accumulator, fp32 sums added in
    slice order) against the same sums built from one-slice calls; and `mirror_cublas`: for every
    row count a split is found with which the outputs are, bit for bit, those of torch's BF16
    matmul on the decoded weight, also where cuBLAS itself splits K (long K, few rows)."""
    from binade_b200.cuda import kernels as ck
    from binade_b200.cuda import r4

    rng = np.random.default_rng(N + K)
    u = weights(rng, (N, K), escapes=False)
    u.reshape(-1)[3::173] = 0x5F80
    m = r4.R4Linear(r4.transcode(packed_arrays(u)))
    w = dev(u).view(torch.bfloat16)
    x = torch.randn((24, K), device="cuda").to(torch.bfloat16)
    # two slices summed by hand from fp32 partials of cuBLAS on the halves (no split there: K / 2 is short or the rows are padded)
    half = K // 2
    if (K // 128) % 2 == 0:
        xp = torch.zeros((256, K), dtype=torch.bfloat16, device="cuda")
        xp[:24] = x
        parts = [torch.mm(xp[:, k0 : k0 + half].contiguous(), w[:, k0 : k0 + half].contiguous().T, out_dtype=torch.float32)[:24] for k0 in (0, half)]
        by_hand = (parts[0] + parts[1]).to(torch.bfloat16)
        assert np.array_equal(words(m.mma_rows(x, split=2)), words(by_hand))
    plan = m.mirror_cublas(rows=(8, 16, 64, 128))
    assert all(v is not None for v in plan.values()), plan
    for M in plan:
        xm = torch.randn((M, K), device="cuda").to(torch.bfloat16)
        assert np.array_equal(words(m.mma_rows(xm)), words(xm @ w.T)), (M, plan[M])
    with pytest.raises(RuntimeError):
        ck.r4_mma(m._a, x, N, K, split=7)  # 7 does not divide the tile count


def test_many_rows_rebuild_path():
    from binade_b200.cuda import r4

    N, K, M = 256, 512, 600  # more rows than the fused kernels take
    rng = np.random.default_rng(5)
    u = weights(rng, (N, K), escapes=False)
    u.reshape(-1)[5::199] = 0x5F80  # 2^64: a rare exponent (escape) that keeps every sum finite
    m = r4.R4Linear(r4.transcode(packed_arrays(u)))
    x = dev(bf16_words(rng.standard_normal((M, K)))).view(torch.bfloat16)
    W = dev(u).view(torch.bfloat16)
    assert torch.equal(m(x), x @ W.T)


@pytest.mark.parametrize("E,N,K,topk", [(8, 176, 704, 4), (8, 704, 176, 4), (6, 96, 384, 2), (16, 64, 520, 8)])
def test_gather(E, N, K, topk):
    from binade_b200.cuda import r4

    rng = np.random.default_rng(N * K)
    u = weights(rng, (E, N, K))
    m = r4.R4Linear(r4.transcode(packed_arrays(u)))
    a = o.pack_r4(u.reshape(E * N, K))
    sel = rng.choice(E, size=topk, replace=False).astype(np.uint32)
    # one shared input row (gate/up), then one input row per selected expert (down)
    for xi in (np.zeros(topk, np.uint32), np.arange(topk, dtype=np.uint32)):
        xw = bf16_words(rng.standard_normal((int(xi.max()) + 1, K)))
        got = m._gather(dev(xw).view(torch.bfloat16), dev(xi), dev(sel), N, N)
        assert np.array_equal(words(got), o.c_r4_gather(a, xw, xi, sel, N, K, N))
    # the upper half of fused rows, and the split form
    half = N // 2
    xw = bf16_words(rng.standard_normal((1, K)))
    xi = np.zeros(topk, np.uint32)
    want = o.c_r4_gather(a, xw, xi, sel, N, K, N)
    got = m._gather(dev(xw).view(torch.bfloat16), dev(xi), dev(sel), N - half, N, half)
    assert np.array_equal(words(got), want[:, half:])
    lo, hi = m._gather(dev(xw).view(torch.bfloat16), dev(xi), dev(sel), N, N, split=half)
    assert np.array_equal(words(lo), want[:, :half]) and np.array_equal(words(hi), want[:, half:])


def test_order_sensitive_gather():
    from binade_b200.cuda import r4

    E, N, K, topk = 8, 48, 704, 4
    u = adversarial(E * N, K).reshape(E, N, K)
    m = r4.R4Linear(r4.transcode(packed_arrays(u)))
    sel = np.array([5, 0, 7, 2], np.uint32)
    got = m._gather(torch.ones((1, K), dtype=torch.bfloat16, device="cuda"), dev(np.zeros(topk, np.uint32)), dev(sel), N, N)
    want = o.c_r4_gather(o.pack_r4(u.reshape(E * N, K)), np.full((1, K), 0x3F80, np.uint16), np.zeros(topk, np.uint32), sel, N, K, N)
    assert np.array_equal(words(got), want)


@pytest.mark.parametrize("tokens,E,topk", [(16, 8, 2), (40, 6, 3), (9, 4, 4)])
def test_grouped_gather_equals_slot_by_slot(tokens, E, topk):
    """Slots grouped by expert (each expert's rows read once for all its tokens) give the bits
    of the slot-by-slot gather, through the kernels and through R4SwitchGLU."""
    from binade_b200.cuda import moe, r4

    n, D = 48, 256
    rng = np.random.default_rng(tokens + E)
    gu = r4.R4Linear(r4.transcode(packed_arrays(weights(rng, (E, 2 * n, D)))))
    dn = r4.R4Linear(r4.transcode(packed_arrays(weights(rng, (E, D, n), escapes=False))))
    x = dev(bf16_words(rng.standard_normal((tokens, D)))).view(torch.bfloat16)
    idx = torch.stack([torch.randperm(E, generator=torch.Generator().manual_seed(t))[:topk] for t in range(tokens)]).cuda()
    ei = idx.reshape(-1).to(torch.int32)
    xi = torch.arange(ei.numel(), dtype=torch.int32, device="cuda") // topk
    g1, u1 = gu._gather(x, xi, ei, 2 * n, 2 * n, split=n)
    g2, u2 = gu._gather_grouped(x, xi, ei, E, tokens, 2 * n, 2 * n, split=n)
    assert np.array_equal(words(g1), words(g2)) and np.array_equal(words(u1), words(u2))
    plain = gu._gather(x, xi, ei, 2 * n, 2 * n)
    assert np.array_equal(words(gu._gather_grouped(x, xi, ei, E, tokens, 2 * n, 2 * n)), words(plain))
    glu = moe.R4SwitchGLU(gu, dn)
    assert tokens * topk >= glu.GROUP_MIN_SLOTS * E  # the grouped path is the one taken
    y = glu(x, idx)
    glu.GROUP_MIN_SLOTS = 1 << 30  # slot by slot
    assert np.array_equal(words(y), words(glu(x, idx)))


def test_padding_slots_are_skipped():
    """A slot whose expert id is NO_EXPERT computes nothing and leaves its output row alone, slot
    by slot and grouped by expert; the other slots are unchanged by its presence."""
    from binade_b200.cuda import kernels as ck
    from binade_b200.cuda import r4

    E, n, K, tokens, topk = 4, 96, 1280, 12, 2
    rng = np.random.default_rng(8)
    m = r4.R4Linear(r4.transcode(packed_arrays(weights(rng, (E, n, K)))))
    x = dev(bf16_words(rng.standard_normal((tokens, K)))).view(torch.bfloat16)
    ei = torch.tensor(rng.integers(0, E, tokens * topk), dtype=torch.int32, device="cuda")
    xi = torch.arange(tokens * topk, dtype=torch.int32, device="cuda") // topk
    plain = m._gather(x, xi, ei, n, n)
    holes = ei.clone()
    holes[[0, 5, 23]] = ck.NO_EXPERT
    keep = torch.ones(tokens * topk, dtype=torch.bool, device="cuda")
    keep[[0, 5, 23]] = False
    for got in (m._gather(x, xi, holes, n, n), m._gather_grouped(x, xi, holes, E, tokens, n, n)):
        assert torch.equal(got[keep].view(torch.int16), plain[keep].view(torch.int16))


def test_convert_swaps_expert_holders():
    from binade_b200.cuda import moe, r4

    rng = np.random.default_rng(4)
    E, n, D = 3, 32, 256
    gu, dn = weights(rng, (E, 2 * n, D)), weights(rng, (E, D, n), escapes=False)

    class Layer(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.experts = moe.BinadeSwitchGLU(packed_arrays(gu), packed_arrays(dn))

    model = Layer()
    with pytest.raises(RuntimeError):
        model.experts(None, None)
    assert r4.convert(model) == 1
    assert isinstance(model.experts, moe.R4SwitchGLU) and (model.experts.E, model.experts.n, model.experts.D) == (E, n, D)
    assert np.array_equal(words(model.experts._gu.dense()), gu) and np.array_equal(words(model.experts._down.dense()), dn)
    x = dev(bf16_words(rng.standard_normal((2, D)))).view(torch.bfloat16)
    idx = torch.tensor([[0, 2], [1, 0]], device="cuda")
    direct = moe.R4SwitchGLU(r4.R4Linear(r4.transcode(packed_arrays(gu))), r4.R4Linear(r4.transcode(packed_arrays(dn))))
    assert torch.equal(model.experts(x, idx).view(torch.int16), direct(x, idx).view(torch.int16))


def test_convert_swaps_holders():
    from binade_b200.cuda import r4

    rng = np.random.default_rng(2)
    u1, u2 = weights(rng, (128, 256)), weights(rng, (64, 128))

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.up = r4.BinadeLinear(packed_arrays(u1))
            self.down = r4.BinadeLinear(packed_arrays(u2))
            self.norm = torch.nn.LayerNorm(4)

    model = torch.nn.Sequential(Block())
    with pytest.raises(RuntimeError):
        model[0].up(torch.zeros(1, 256))
    assert r4.convert(model) == 2
    assert isinstance(model[0].up, r4.R4Linear) and (model[0].up.N, model[0].up.K, model[0].up.T) == (128, 256, 2)
    assert np.array_equal(words(model[0].down.dense()), u2)
    hs = r4.holders(GOLDEN / "packed_model" / "packed")
    assert set(hs) == {"model.embed_tokens.weight", "model.layers.0.self_attn.q_proj.weight", "model.layers.0.experts.gate_up_proj", "lm_head.weight"}
    a = r4.transcode(hs["lm_head.weight"])
    assert a["shape"] == (300, 256)


def test_switch_glu_matches_oracle():
    """MoE decode step: fused gate/up gather, SwiGLU, down gather, against the oracle's products."""
    from binade_b200.cuda import moe, r4

    E, n, D, tokens, k = 8, 96, 256, 3, 4
    rng = np.random.default_rng(21)
    gu, dn = weights(rng, (E, 2 * n, D)), weights(rng, (E, D, n), escapes=False)
    gu.reshape(-1)[::997] = 0x3C00  # keep gate/up finite: no Inf patterns in this test
    gu.reshape(-1)[5::199] = 0x5F80
    m = moe.R4SwitchGLU(r4.R4Linear(r4.transcode(packed_arrays(gu))), r4.R4Linear(r4.transcode(packed_arrays(dn))))
    assert (m.E, m.n, m.D) == (E, n, D)
    xw = bf16_words(rng.standard_normal((tokens, D)) * 0.1)
    idx = np.stack([rng.choice(E, size=k, replace=False) for _ in range(tokens)]).astype(np.int64)
    y = m(dev(xw).view(torch.bfloat16), torch.from_numpy(idx).cuda())
    assert y.shape == (tokens, k, D)
    a_gu, a_dn = o.pack_r4(gu.reshape(E * 2 * n, D)), o.pack_r4(dn.reshape(E * D, n))
    ei = idx.reshape(-1).astype(np.uint32)
    xi = (np.arange(ei.size) // k).astype(np.uint32)
    both = o.c_r4_gather(a_gu, xw, xi, ei, 2 * n, D, 2 * n)
    gate, up = torch.from_numpy(both[:, :n].view(np.int16).copy()).view(torch.bfloat16), torch.from_numpy(both[:, n:].view(np.int16).copy()).view(torch.bfloat16)
    h = words(moe.swiglu(up, gate))
    want = o.c_r4_gather(a_dn, h, np.arange(ei.size, dtype=np.uint32), ei, D, n, D)
    assert np.array_equal(words(y).reshape(-1, D), want)


def test_zz_device_status_is_clean():
    """No kernel of this run gave up a bounded wait (collected last in this file)."""
    import ctypes

    from binade_b200 import _native

    st = ctypes.c_int(-1)
    _native.call("cuda", "bn_device_status", ctypes.byref(st))
    assert st.value == 0
