"""The CPU oracle (numpy and C restatements) against vectors computed by the reference itself.

This is what pins parity: every GPU test compares against the oracle, and the oracle is
compared here with the reference's outputs (tests/golden, see make_golden.py) and with the
reference's hand-computed stream (its tests/test_rice.py:50-56)."""

import numpy as np
import pytest

from conftest import golden
from oracle import oracle as o

CODEC = golden("codec_cases.npz")
CASES = [c for c in CODEC if "exps" in CODEC[c]]


@pytest.mark.parametrize("case", CASES)
def test_rank_table_and_rice_encode(case):
    g = CODEC[case]
    hist = np.bincount(g["exps"].ravel(), minlength=256)
    for table, rank in (o.np_rank_table(hist), o.c_rank_table(hist)):
        assert np.array_equal(table, g["table"]) and np.array_equal(rank, g["rank"])
    ranks = g["rank"][g["exps"]]
    for meta, bits, roff in (o.np_rice_encode_ranks(ranks), o.c_rice_encode_ranks(ranks)):
        assert np.array_equal(meta, g["meta"])
        assert np.array_equal(bits, g["bits"])
        assert np.array_equal(roff, g["roff"])


@pytest.mark.parametrize("case", CASES)
def test_rice_decode(case):
    g = CODEC[case]
    K = g["exps"].shape[1]
    for ranks, end in (o.np_rice_decode_ranks(g["meta"], g["bits"], g["roff"], K), o.c_rice_decode_ranks(g["meta"], g["bits"], g["roff"], K)):
        assert np.array_equal(ranks, g["ranks"])
        assert np.array_equal(end, g["end"])
    assert np.array_equal(o.np_rice_decode(g["table"], g["meta"], g["bits"], g["roff"], *g["exps"].shape), g["exps"])


def test_hand_computed_stream():
    """Ranks [0,1,5,2]: k = 1 (4 low + 6 unary bits); low plane 0110, plane 0 0011, plane 1 10."""
    stream = [0, 1, 1, 0, 0, 0, 1, 1, 1, 0]
    word = sum(b << i for i, b in enumerate(stream))
    for meta, bits, roff in (o.np_rice_encode_ranks(np.array([[0, 1, 5, 2]])), o.c_rice_encode_ranks(np.array([[0, 1, 5, 2]]))):
        assert meta.tolist() == [1 | 2 << 2] and roff.tolist() == [0] and bits.tolist() == [word]
    g = CODEC["by_hand"]
    assert g["meta"].tolist() == [1 | 2 << 2] and g["bits"].tolist() == [word]


def test_rank_ties_and_absent_exponents():
    g = CODEC["ties"]
    for table, rank in (o.np_rank_table(g["hist"]), o.c_rank_table(g["hist"])):
        assert np.array_equal(table, g["table"]) and np.array_equal(rank, g["rank"])
    assert g["table"][:5].tolist() == [120, 3, 9, 121, 200] and not g["table"][5:].any()


def test_k_and_qmax_limits():
    """All ranks 255: k must be >= 2 so that qmax = 255 >> k fits 6 bits (reference tests/test_rice.py:89-93)."""
    for meta, _, _ in (o.np_rice_encode_ranks(np.full((1, 128), 255)), o.c_rice_encode_ranks(np.full((1, 128), 255))):
        k, qmax = meta[0] & 3, meta[0] >> 2
        assert k >= 2 and qmax == 255 >> k and qmax <= 63


def test_split_join_every_pattern():
    w = np.arange(1 << 16, dtype=np.uint32).astype(np.uint16)
    raw, exps = o.np_split(w)
    assert np.array_equal(o.np_join(raw, exps), w)
    g = golden("config1_small.npz")[""]
    raw, exps = o.np_split(g["w"])
    assert np.array_equal(raw, g["raw"]) and np.array_equal(exps, g["exps"])


def test_config1_small_parts():
    g = golden("config1_small.npz")[""]
    raw, table, ranks = o.c_ranks_of(g["w"])
    assert np.array_equal(raw, g["raw"]) and np.array_equal(table, g["table"])
    assert np.array_equal(ranks, g["rank"][g["exps"]])
    meta, bits, roff = o.c_rice_encode_ranks(ranks)
    assert np.array_equal(meta, g["meta"]) and np.array_equal(bits, g["bits"]) and np.array_equal(roff, g["roff"])
    back, end = o.c_rice_decode_ranks(meta, bits, roff, g["w"].shape[1])
    assert np.array_equal(o.np_join(raw, table[back]), g["w"])


@pytest.mark.parametrize("case", list(golden("r4_layout.npz")))
def test_r4_layout(case):
    g = golden("r4_layout.npz")[case]
    ranks = g["rank"][o.np_split(g["w"])[1]]
    for a in (o.np_r4_transcode(ranks, g["table"]), o.c_r4_transcode(ranks, g["table"])):
        for k in ("codes", "flags", "esc", "row_esc"):
            assert np.array_equal(a[k], g[k]), k
        a = dict(a, raw=g["raw"], table=g["table"])
        R, K = g["w"].shape
        assert np.array_equal(o.np_r4_dense(a, R, K), g["w"])
        assert np.array_equal(o.c_r4_dense(a, R, K), g["w"])
    assert g["flags"].any() and g["esc"].size > 1


def test_truncated_stream_is_rejected():
    g = CODEC["geometric_20x1000"]
    with pytest.raises(ValueError):
        o.np_rice_decode(g["table"], g["meta"], g["bits"][:-1], g["roff"], *g["exps"].shape)
    _, end = o.c_rice_decode_ranks(g["meta"], g["bits"][:-1], g["roff"], 1000)
    nxt = np.append(g["roff"][1:].astype(np.int64), g["bits"].size - 1)
    assert np.any((end + 31) >> 5 != nxt)


def test_same_order_rows_numpy_equals_c():
    rng = np.random.default_rng(7)
    for N, K in ((24, 704), (16, 256), (9, 100), (5, 4)):
        w = (rng.standard_normal((N, K)).astype(np.float32) * 0.02).view(np.uint32) >> 16
        x = rng.standard_normal((3, K)).astype(np.float32).view(np.uint32) >> 16
        w, x = w.astype(np.uint16), x.astype(np.uint16)
        assert np.array_equal(o.np_rows_same_order(x, w), o.c_dense_rows(x, w))
        a = o.pack_r4(w)
        assert np.array_equal(o.c_r4_matvec(a, x[0], N, K), o.c_dense_rows(x[:1], w)[0])


def test_summation_order_is_observable():
    """+2^25, ones, -2^25 on one lane: in order the ones vanish (sum 0); another order keeps some."""
    K = 1024
    w = np.zeros((1, K), np.float32)
    w[0, 0], w[0, 128 * 7] = 2.0**25, -(2.0**25)
    w[0, 128:896:128] = 1.0
    wb = (w.view(np.uint32) >> 16).astype(np.uint16)
    ones = np.full((1, K), 0x3F80, np.uint16)
    assert o.c_dense_rows(ones, wb)[0, 0] == 0
    assert float(w.astype(np.float64).sum()) == 6.0


@pytest.mark.parametrize("name", ["bench_16x512", "bench_8x128", "wide_6x1280"])
def test_format1_oracle_against_reference_vectors(name):
    """The numpy restatement of format 1 (binade/format.py) writes the reference's own encode
    output for the golden tensors and decodes it back; a stream that is too short is refused."""
    f1, lay = golden("format1.npz"), golden("r4_layout.npz")
    w, table, rank = lay[name]["w"], lay[name]["table"], lay[name]["rank"]
    raw, exps = o.np_split(w)
    meta, idx, esc = o.np_f1_encode(exps, table, rank)
    assert np.array_equal(meta, f1[name]["meta"]) and np.array_equal(idx, f1[name]["idx"]) and np.array_equal(esc, f1[name]["esc"])
    back = o.np_f1_decode(meta, idx, esc, table, *w.shape)
    assert np.array_equal(back, exps) and np.array_equal(o.np_join(raw, back), w)
    with pytest.raises(ValueError):
        o.np_f1_decode(meta, idx, esc[:-1], table, *w.shape)
    with pytest.raises(ValueError):
        o.np_f1_decode(meta, idx[:-4], esc, table, *w.shape)


def test_esc_columns_restatement_against_a_plain_loop():
    """oracle.esc_columns (the definition the GPU builder is checked against) itself, against a
    weight-by-weight walk of the R4 arrays on a tensor dense with escapes and a short last tile."""
    rng = np.random.default_rng(5)
    R, K = 9, 272
    u = rng.integers(0, 1 << 16, size=(R, K), dtype=np.uint16)
    a = o.pack_r4(u)
    esc_cols, col_esc = o.esc_columns(a)
    T = -(-K // 128)
    codes = a["codes"].reshape(R, T * 32)
    n = a["esc"].size - 1
    assert n > 100 and esc_cols.size == n + 8 and not esc_cols[n:].any()
    for r in range(R):
        cursor = int(a["row_esc"][r])
        buckets = [[] for _ in range(16)]
        for k in range(T * 128):
            if (int(codes[r, k // 4]) >> (4 * (k % 4))) & 15 == 15:
                buckets[(k % 128) // 8].append(int(a["esc"][cursor]))
                cursor += 1
        start = 0
        for c in range(16):
            assert int(col_esc[r, c]) == start, (r, c)
            at = int(a["row_esc"][r]) + start
            assert list(esc_cols[at : at + len(buckets[c])]) == buckets[c], (r, c)
            start += len(buckets[c])
