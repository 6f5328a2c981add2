"""Row sharding across ranks, on CPU: the cuts (index arithmetic) against the oracle, and the
gather wiring with two gloo ranks (the local product is the oracle here: the CUDA kernels cannot
run without a GPU, and the sharded module only adds the cut and the collective around them)."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from binade_b200 import pack
from binade_b200.cuda import dist as bd
from oracle import oracle as o


def _weights(shape, seed=0):
    rng = np.random.default_rng(seed)
    w = rng.standard_normal(shape).astype(np.float32) * 0.02
    w[rng.random(shape) < 5e-3] *= 64
    return (w.view(np.uint32) >> 16).astype(np.uint16)


def test_row_range_covers_rows_once():
    for N in (0, 1, 7, 8, 100, 4097):
        for world in (1, 2, 3, 8):
            spans = [bd.row_range(N, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == N
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert max(b - a for a, b in spans) - min(b - a for a, b in spans) <= 1
    with pytest.raises(ValueError):
        bd.row_range(8, 2, 2)


@pytest.mark.parametrize("N,K,world", [(37, 704, 2), (64, 256, 4), (10, 100, 3), (5, 128, 8)])
def test_shard_packed_decodes_to_its_rows(N, K, world):
    u = _weights((N, K), seed=N)
    p = pack.pack(u)
    got = []
    for rank in range(world):
        s = bd.shard_packed(p, rank, world)
        r0, r1 = bd.row_range(N, rank, world)
        assert s["shape"] == (r1 - r0, K) and s["meta"].size == (r1 - r0) * -(-K // 128)
        if r1 > r0:
            ranks, end = o.c_rice_decode_ranks(s["meta"], s["bits"], s["roff"], K)
            nxt = np.append(s["roff"][1:].astype(np.int64), s["bits"].size)
            assert np.array_equal((end + 31) >> 5, nxt)
            got.append(o.np_join(s["raw"], s["table"][ranks]))
    assert np.array_equal(np.concatenate(got), u)


@pytest.mark.parametrize("N,K,world", [(37, 704, 2), (64, 256, 4), (9, 128, 8)])
def test_shard_r4_matches_oracle_rows(N, K, world):
    u = _weights((N, K), seed=K)
    a = o.pack_r4(u)
    _, table, ranks = o.c_ranks_of(u)  # the tensor's own table: a shard keeps it
    t = {k: torch.from_numpy(v.view(np.int16) if v.dtype == np.uint16 else v.view(np.int32) if v.dtype == np.uint32 else v) for k, v in a.items() if k != "shape"}
    t["raw"] = t["raw"].reshape(N, K)
    pieces = []
    for rank in range(world):
        s = bd.shard_r4(t, rank, world)
        r0, r1 = bd.row_range(N, rank, world)
        want = o.c_r4_transcode(ranks[r0:r1], table) if r1 > r0 else None
        if want is None:
            assert s["raw"].shape[0] == 0 and s["esc"].numel() == 1
            continue
        assert np.array_equal(s["codes"].numpy().view(np.uint16), want["codes"])
        assert np.array_equal(s["flags"].numpy(), want["flags"])
        assert np.array_equal(s["esc"].numpy(), want["esc"])
        assert np.array_equal(s["row_esc"].numpy().view(np.uint32), want["row_esc"])
        pieces.append(s["raw"].numpy())
    assert np.array_equal(np.concatenate(pieces), a["raw"].reshape(N, K))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, N: int, K: int, out_dir: str):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    u = _weights((N, K), seed=3)
    x = _weights((1, K), seed=4)
    shard = bd.shard_packed(pack.pack(u), rank, world)
    ranks, _ = o.c_rice_decode_ranks(shard["meta"], shard["bits"], shard["roff"], K)
    w_local = o.np_join(shard["raw"], shard["table"][ranks])

    def local(xt):  # stands for R4Linear(transcode(shard)) on this rank's GPU
        y = o.c_dense_rows(xt.view(torch.int16).numpy().view(np.uint16).reshape(-1, K), w_local)
        return torch.from_numpy(y.view(np.int16)).view(torch.bfloat16).reshape(*xt.shape[:-1], -1)

    m = bd.RowShardedLinear(local, N)
    y = m(torch.from_numpy(x.view(np.int16)).view(torch.bfloat16))
    np.save(os.path.join(out_dir, f"y{rank}.npy"), y.view(torch.int16).numpy().view(np.uint16))
    dist.destroy_process_group()


@pytest.mark.parametrize("N", [64, 37])
def test_row_sharded_linear_two_gloo_ranks(tmp_path, N):
    K, world = 256, 2
    mp.spawn(_rank_main, args=(world, _free_port(), N, K, str(tmp_path)), nprocs=world, join=True)
    want = o.c_dense_rows(_weights((1, K), seed=4), _weights((N, K), seed=3))
    for rank in range(world):
        assert np.array_equal(np.load(tmp_path / f"y{rank}.npy"), want), rank


def _group_main(rank: int, world: int, port: int, out_dir: str):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    K, Ns = 128, (32, 8, 8)
    x = _weights((3, K), seed=9)

    def local_of(N, seed):
        r0, r1 = bd.row_range(N, rank, world)
        w_local = _weights((N, K), seed=seed)[r0:r1]

        def local(xt):
            y = o.c_dense_rows(xt.view(torch.int16).numpy().view(np.uint16).reshape(-1, K), w_local)
            return torch.from_numpy(y.view(np.int16)).view(torch.bfloat16).reshape(*xt.shape[:-1], -1)

        return local

    g = bd.RowShardedGroup([local_of(N, 20 + i) for i, N in enumerate(Ns)], Ns)
    ys = g(torch.from_numpy(x.view(np.int16)).view(torch.bfloat16))
    for i, y in enumerate(ys):
        np.save(os.path.join(out_dir, f"g{rank}_{i}.npy"), y.view(torch.int16).numpy().view(np.uint16))
    # the deferred form: local slices of a one-row input, gathered by one collective
    x1 = torch.from_numpy(x[:1].view(np.int16)).view(torch.bfloat16)
    late = bd.gather_all(g(x1, gather=False))
    same = all(torch.equal(a.view(torch.int16), b.view(torch.int16)) for a, b in zip(late, g(x1)))
    with open(os.path.join(out_dir, f"late{rank}"), "w") as f:
        f.write("1" if same and len(late) == len(Ns) else "0")
    dist.destroy_process_group()


def test_row_sharded_group_two_gloo_ranks(tmp_path):
    """Three projections of one input, one all-gather: every full output equals the unsharded
    product on every rank."""
    world = 2
    mp.spawn(_group_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    x = _weights((3, 128), seed=9)
    for i, N in enumerate((32, 8, 8)):
        want = o.c_dense_rows(x, _weights((N, 128), seed=20 + i))
        for rank in range(world):
            assert np.array_equal(np.load(tmp_path / f"g{rank}_{i}.npy"), want), (rank, i)
    assert [(tmp_path / f"late{r}").read_text() for r in range(world)] == ["1", "1"]  # gather_all of the local slices


def _ep_case():
    E, D, tokens, k = 8, 16, 6, 3
    g = torch.Generator().manual_seed(9)
    x = torch.randn((tokens, D), generator=g).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(tokens)])
    idx[5, 2] = -1  # a padding slot: routed nowhere, output zero
    table = torch.randn((E, D), generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)  # a toy "expert": y = x * table[e]
    return E, D, x, idx, table


def _ep_main(rank: int, world: int, port: int, out_dir: str):
    import torch.distributed as dist

    from binade_b200.cuda import moe

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    E, D, x, idx, table = _ep_case()
    mine = slice(rank * x.shape[0] // world, (rank + 1) * x.shape[0] // world)  # this rank's share of the batch

    def local_slots(xf, xi, ei_local):  # stands for R4SwitchGLU.slots over this rank's experts; padding slots untouched
        out = torch.full((ei_local.numel(), D), 7.0, dtype=torch.bfloat16)
        real = ei_local >= 0
        out[real] = xf[xi[real].long()] * table[ei_local[real].long() + rank * (E // world)]
        return out

    y = moe.ExpertParallelGLU(local_slots, E, D, rank, world)(x[mine], idx[mine])
    torch.save(y, os.path.join(out_dir, f"y{rank}.pt"))
    dist.destroy_process_group()


def test_expert_parallel_two_gloo_ranks(tmp_path):
    """Every slot's input row reaches the rank owning its expert (all-to-all), is computed there
    once, and its output comes back to the slot's place on the rank that holds the token."""
    world = 2
    mp.spawn(_ep_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    E, D, x, idx, table = _ep_case()
    want = x[:, None, :] * table[idx.clamp(min=0)]
    want[idx < 0] = 0
    for r in range(world):
        mine = slice(r * x.shape[0] // world, (r + 1) * x.shape[0] // world)
        assert torch.equal(torch.load(tmp_path / f"y{r}.pt"), want[mine]), r
