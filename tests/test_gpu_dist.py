"""Row-sharded linear on two GPUs (NCCL): gathered output equals the single-GPU product bit for
bit. Skipped on a box with one GPU."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _rank_main(rank: int, world: int, port: int, N: int, K: int, out_dir: str):
    import torch.distributed as dist

    from binade_b200 import pack
    from binade_b200.cuda import dist as bd
    from binade_b200.cuda import kernels as ck
    from binade_b200.cuda import r4
    from test_gpu_parity import bf16_words, weights

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    rng = np.random.default_rng(5)
    u = weights(rng, (N, K), escapes=False)
    u.reshape(-1)[7::211] = 0x5F80  # rare exponent: escapes, finite sums
    xw = bf16_words(rng.standard_normal((1, K)))
    p = pack.pack(u)
    x = ck.to_device(xw).view(torch.bfloat16)
    local = r4.R4Linear(r4.transcode(bd.shard_packed(p, rank, world)))
    y = bd.RowShardedLinear(local, N)(x)
    cut = r4.R4Linear(bd.shard_r4(r4.transcode(p), rank, world))  # the same rows, cut after expansion
    y2 = bd.RowShardedLinear(cut, N)(x)
    full = r4.R4Linear(r4.transcode(p))(x)
    ok = torch.equal(y.view(torch.int16), full.view(torch.int16)) and torch.equal(y2.view(torch.int16), full.view(torch.int16))
    # two projections of one input as a group (one launch, one exchange), and the deferred form:
    # local slices of two groups gathered by one collective, through the peer-store kernel and NCCL
    if N % world == 0:
        ex = bd.make_exchange(max_bytes=8 * N)
        for exchange in (ex, None):
            grp = bd.RowShardedGroup([local, cut], [N, N], exchange=exchange)
            a, b = grp(x)
            ok = ok and torch.equal(a.view(torch.int16), full.view(torch.int16)) and torch.equal(b.view(torch.int16), full.view(torch.int16))
            both = bd.gather_all(grp(x, gather=False) + grp(x, gather=False), exchange=exchange)
            ok = ok and len(both) == 4 and all(torch.equal(t.view(torch.int16), full.view(torch.int16)) for t in both)
            # the same collective on a stream of its own (the small-block kernel), joined afterwards
            side = torch.cuda.Stream()
            beside = bd.gather_all(grp(x, gather=False), exchange=exchange, stream=side)
            torch.cuda.current_stream().wait_stream(side)
            ok = ok and len(beside) == 2 and all(torch.equal(t.view(torch.int16), full.view(torch.int16)) for t in beside)
        if ex is not None:
            ex.check()
    with open(os.path.join(out_dir, f"ok{rank}"), "w") as f:
        f.write("1" if ok else "0")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("N,K", [(512, 3840), (301, 704)])
def test_row_sharded_linear_two_gpus(tmp_path, N, K):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_rank_main, args=(2, port, N, K, str(tmp_path)), nprocs=2, join=True)
    assert [(tmp_path / f"ok{r}").read_text() for r in range(2)] == ["1", "1"]


def _decoder_main(rank: int, world: int, port: int, out_dir: str):
    import torch.distributed as dist

    from binade_b200.cuda.llama import Decoder
    from test_gpu_decoder import tiny

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    prompt = torch.randint(0, 512, (6,), device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    sharded, _ = Decoder(tiny(), kind="r4", rank=rank, world=world).generate(prompt, 12, use_graph=True)
    single, _ = Decoder(tiny(), kind="r4").generate(prompt, 12, use_graph=True)
    with open(os.path.join(out_dir, f"ok{rank}"), "w") as f:
        f.write("1" if torch.equal(sharded, single) else "0")
    dist.barrier()
    dist.destroy_process_group()


def test_row_sharded_decoder_two_gpus(tmp_path):
    """Row sharding keeps every output's summation order: greedy tokens equal the 1-GPU run."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_decoder_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert [(tmp_path / f"ok{r}").read_text() for r in range(2)] == ["1", "1"]


def _push_main(rank: int, world: int, port: int, out_dir: str):
    import torch.distributed as dist

    from binade_b200 import _native
    from binade_b200.cuda import dist as bd

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ex = bd.PushGather(max_bytes=1 << 16)
    ok = True
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    for shape in ((1, 1920), (3, 200), (1, 8), (5, 33)):  # the last one needs padding to 16 bytes
        flat = torch.randn(shape, device="cuda", generator=g).to(torch.bfloat16)
        want = torch.empty((world * shape[0], shape[1]), dtype=torch.bfloat16, device="cuda")
        dist.all_gather_into_tensor(want, flat)
        got = ex(flat).clone()
        ok = ok and torch.equal(got.view(torch.int16), want.view(world, *shape).view(torch.int16))
    # a captured graph replays the exchange (the call number lives on the device)
    flat = torch.full((1, 64), float(rank + 1), device="cuda", dtype=torch.bfloat16)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        ex(flat)
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            out = ex(flat).clone()
    for i in range(3):
        flat.fill_(float(10 * i + rank + 1))
        graph.replay()
        torch.cuda.synchronize()
        ok = ok and all(bool((out[r] == 10 * i + r + 1).all()) for r in range(world))
    # the grouped sharded hook over the exchange equals the NCCL one
    locals_ = [lambda x, s=s: (x[..., : 16 * (s + 1)] * (rank + 1)).contiguous() for s in range(2)]
    x = torch.randn((1, 64), device="cuda", generator=g).to(torch.bfloat16)
    dist.broadcast(x, 0)
    a = bd.RowShardedGroup(locals_, [16 * world, 32 * world], exchange=bd.PushGather(max_bytes=4096))(x)
    b = bd.RowShardedGroup(locals_, [16 * world, 32 * world])(x)
    ok = ok and all(torch.equal(p, q) for p, q in zip(a, b))
    status = _native.C.c_int(-1)
    _native.call("cuda", "bn_device_status", _native.C.byref(status))
    ok = ok and status.value == 0
    with open(os.path.join(out_dir, f"ok{rank}"), "w") as f:
        f.write("1" if ok else "0")
    dist.barrier()
    dist.destroy_process_group()


def test_push_gather_two_gpus(tmp_path):
    """The peer-store all-gather kernel returns what NCCL's all-gather returns, also when
    replayed from a CUDA graph and under the grouped sharded hook."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_push_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert [(tmp_path / f"ok{r}").read_text() for r in range(2)] == ["1", "1"]


def _ep_main(rank: int, world: int, port: int, out_dir: str):
    import torch.distributed as dist

    from binade_b200.cuda import moe, r4

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    E, n, D, k = 8, 128, 768, 3
    g = torch.Generator(device="cuda").manual_seed(11)
    gu = (torch.randn((E, 2 * n, D), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    dn = (torch.randn((E, D, n), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    per = E // world
    whole = moe.R4SwitchGLU(r4.R4Linear(r4.from_dense(gu)), r4.R4Linear(r4.from_dense(dn)))
    local = moe.R4SwitchGLU(r4.R4Linear(r4.from_dense(gu[rank * per : (rank + 1) * per].contiguous())), r4.R4Linear(r4.from_dense(dn[rank * per : (rank + 1) * per].contiguous())))
    ep = moe.ExpertParallelGLU(local.slots, E, D, rank, world)
    ok = True
    for tokens in (2, 8, 40):  # per rank: slot by slot, then grouped by expert
        x = torch.randn((world * tokens, D), device="cuda", generator=g).to(torch.bfloat16)
        idx = torch.stack([torch.randperm(E, device="cuda", generator=g)[:k] for _ in range(world * tokens)])
        idx[1, 0] = -1  # a padding slot
        mine = slice(rank * tokens, (rank + 1) * tokens)
        y = ep(x[mine], idx[mine])
        want = whole(x[mine], idx[mine].clamp(min=0))
        want[idx[mine] < 0] = 0
        ok = ok and torch.equal(y.view(torch.int16), want.view(torch.int16))
    with open(os.path.join(out_dir, f"ep{rank}"), "w") as f:
        f.write("1" if ok else "0")
    dist.barrier()
    dist.destroy_process_group()


def test_expert_parallel_two_gpus(tmp_path):
    """Experts and tokens split over two GPUs, all-to-all dispatch and combine: every output is
    bit-identical to the single-GPU layer over all experts."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_ep_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert [(tmp_path / f"ep{r}").read_text() for r in range(2)] == ["1", "1"]
