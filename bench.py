"""Benchmark of the Binade hot path on B200: load-time Rice->R4 expansion and the batch-1 fused
R4-decode matvec on 12B-class shapes (seven projection matrices of one decoder layer).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one token's seven matvecs (q, k, v, o, gate, up, down) over weights resident in HBM
in the R4 layout, issued as a decoder layer issues them: projections that share their input go
in one launch (q k v | o | gate up | down). Steps rotate over several copies of the weights so
that no step finds its weights in L2 (one copy is 338 MB, L2 is 126 MB). The metric is the
compressed bytes the kernels stream per second. The last stdout line is one JSON object.

Before anything is timed, every matrix of the workload is checked at full size against the CPU
oracle: the expander's arrays, the dense decode and the matvec, bit for bit.

With N > 1 (launched by torch.distributed.run, one rank per GPU) every rank holds its own row
shard of an N-times taller layer (same per-GPU work: weak scaling) and all-gathers the step's
seven output slices with one exchange per step inside the timed region, on a second stream so
that it overlaps the next step's products; the gathered vectors are checked on every rank,
before the timing (eager steps) and after it (what the timed graphs left in their buffers).
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SHAPES = [("q", 4096, 3840), ("k", 2048, 3840), ("v", 2048, 3840), ("o", 3840, 4096), ("gate", 15360, 3840), ("up", 15360, 3840), ("down", 3840, 15360)]
WORKLOAD = "config2: Rice->R4 expansion + batch-1 fused R4 matvec, 7 matrices of a 12B-class layer (q 4096x3840, k/v 2048x3840, o 3840x4096, gate/up 15360x3840, down 3840x15360), N(0,0.02) BF16 with 0.1% x64 outliers, x ~ N(0,1)"
METRIC, UNIT = "r4_matvec_hbm_gbs", "GB/s"
NOMINAL_HBM_GBS = 8000.0
GRAPH_ROUNDS = 8  # a timed graph holds this many steps per weight copy
# DRAM bytes (read + write) over algorithmic bytes of one matvec launch, from one ncu capture of
# the batch-1 kernel on the gate matrix (89.6 MB read + 4.9 MB written for 89.06 MB); the JSON
# line labels the figure as assumed from that capture, scaled to the average launch by bytes.
NCU_TRAFFIC_RATIO = 94.5 / 89.06
OUTLIERS = 1e-3  # fraction of weights scaled x64 (the benchmark's distribution)
GROUPS = (("q", "k", "v"), ("o",), ("gate", "up"), ("down",))  # projections sharing an input: one launch each


def synthetic_weight(name: str, n: int, k: int, seed_base: int = 0) -> np.ndarray:
    """BF16 words [n, k]: N(0, 0.02), 0.1 % of entries scaled x64, seeded per matrix."""
    import torch

    seed = seed_base * 1000 + sum(ord(c) for c in name) + n + k
    g = torch.Generator().manual_seed(seed)
    w = torch.randn((n, k), generator=g) * 0.02
    w = torch.where(torch.rand((n, k), generator=g) < OUTLIERS, w * 64, w)
    return w.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def synthetic_input(k: int, seed: int) -> np.ndarray:
    import torch

    g = torch.Generator().manual_seed(77 + seed)
    return torch.randn(k, generator=g).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def measured_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "source": "measured (MEASURED_PEAKS.json)"}
    return {"hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi in the background during the timed region (reads settings, changes none)."""

    FIELDS = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, gpu: int):
        self.gpu, self.proc, self.path = gpu, None, None

    def __enter__(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50", "-i", str(self.gpu)], stdout=f, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.12)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if not self.path or not os.path.exists(self.path):
            return out
        sm, mx, reasons = [], [], set()
        for line in Path(self.path).read_text().splitlines():
            f = [s.strip() for s in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            out.update(sm_mhz=float(np.median(sm)), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


# ----------------------------------------------------------------------------- CPU arm
def cpu_r4_layer(seed_base: int, names=None):
    """The layer's R4 arrays built on the host by the oracle (for the CPU arms only)."""
    from oracle import oracle as o

    mats = []
    for name, n, k in SHAPES:
        if names and name not in names:
            continue
        a = o.pack_r4(synthetic_weight(name, n, k, seed_base))
        mats.append((name, n, k, a, sum(a[key].nbytes for key in ("raw", "codes", "flags", "esc", "table", "row_esc")) + 2 * k + 2 * n))
    return mats


def cpu_step(mats, xs, frac: float = 1.0):
    """One CPU step over the first `frac` of every matrix's rows; returns the bytes it streamed."""
    from oracle import oracle as o

    z = np.zeros(1, np.uint32)
    done = 0
    for _, n, k, a, nbytes in mats:
        rows = max(1, int(n * frac))
        o.c_r4_gather(a, xs[k], z, z, rows, k, 0, 0)
        done += nbytes * rows / n
    return done


def cpu_cores() -> int:
    return len(os.sched_getaffinity(0))


def run_reference(args) -> dict:
    """The CPU arm: the oracle's C restatement of the same step on all host threads. The
    reference project has no CPU matvec (its CPU code is the numpy codec) and its GPU kernels
    need MLX, which this box lacks, so the C port of its kernel semantics stands in. Each step
    covers the same fraction of every matrix's rows, sized so the run ends within about a minute."""
    from oracle import oracle as o

    threads = o.set_threads(cpu_cores())  # a multi-process launcher caps OMP_NUM_THREADS at 1
    mats = cpu_r4_layer(0)
    xs = {k: synthetic_input(k, 0) for k in {k for _, _, k in SHAPES}}
    t0 = time.perf_counter()
    cpu_step(mats, xs, 1 / 32)
    full = (time.perf_counter() - t0) * 32
    frac = min(1.0, 60.0 / (full * (args.steps + args.warmup)))
    for _ in range(args.warmup):
        cpu_step(mats, xs, frac)
    t0, done = time.perf_counter(), 0.0
    for _ in range(args.steps):
        done += cpu_step(mats, xs, frac)
    dt = time.perf_counter() - t0
    val = done / dt / 1e9
    base = {"value": val, "unit": UNIT, "cores": threads, "kind": "port", "sample": f"every step: the first {frac:.4f} of the rows of each of the 7 matrices, C oracle with OpenMP over rows"}
    return {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 weights (R4 coded), fp32 accumulate",
        "data": "synthetic", "config": {"workload": WORKLOAD, "where": "host CPU", "row_fraction_per_step": frac}, "cpu_baseline": base,
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0,
    }  # fmt: skip


# ----------------------------------------------------------------------------- GPU arm
def run_ours(args) -> dict | None:
    import torch

    import ctypes

    from binade_b200 import _native, pack
    from binade_b200.cuda import kernels as ck
    from binade_b200.cuda import r4

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        import datetime

        # a short timeout: a rank that dies or falls out of step ends the run instead of holding the GPUs
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=120))
    dev = torch.device("cuda", local)
    copies = args.copies
    t_start = time.perf_counter()

    def note(msg: str):  # progress on stderr: a stalled run shows where it stopped
        print(f"[bench rank {rank} +{time.perf_counter() - t_start:6.1f}s] {msg}", file=sys.stderr, flush=True)

    # ---- build: host Rice encode (product packer), device expand (timed), R4 resident; every
    # matrix is checked at full size against the CPU oracle before it is used: the expander's
    # four arrays, the dense decode (against the source words) and the batch-1 product
    from oracle import oracle as o

    o.set_threads(cpu_cores())
    layers, expand_ms, expand_bytes, host_pack_s, bits_file, bits_r4 = [], 0.0, 0, 0.0, 0, 0
    columns_ms = 0.0  # building the column-ordered escapes, per layer
    gpu_pack_s = 0.0  # the GPU Rice encoder on the same matrices (wall clock with its two host reads)
    numel = 0
    parity = {"matrices": 0, "expander_arrays": "bit-identical to the oracle", "escape_columns": "identical to their definition restated in numpy", "gpu_encoder": "file arrays identical to the host packer's", "dense_decode": "bit-identical to the source words", "matvec": "bit-identical to the oracle (documented order)"}
    xs_host = {k: synthetic_input(k, 0) for k in {k for _, _, k in SHAPES}}  # every rank multiplies the same input, as row-sharded layers do
    for name, n, k in SHAPES:
        u = synthetic_weight(name, n, k, rank)
        t0 = time.perf_counter()
        p = pack.pack(u)
        host_pack_s += time.perf_counter() - t0
        d = {key: ck.to_device(p[key]) for key in ("raw", "table", "meta", "bits", "roff")}
        torch.cuda.synchronize()
        # the same arrays from the GPU encoder (words already on the device), checked and timed
        u_dev = ck.to_device(u.view(np.int16))
        enc = ck.rice_encode(u_dev)
        if not all(torch.equal(enc[key].reshape(-1).view(torch.uint8), d[key].reshape(-1).view(torch.uint8)) for key in ("raw", "table", "meta", "bits", "roff")):
            raise SystemExit(f"bench: GPU Rice encoder output of {name} differs from the host packer's; refusing to report a number")
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        ck.rice_encode(u_dev)
        torch.cuda.synchronize()
        gpu_pack_s += time.perf_counter() - t0
        del enc, u_dev
        a = r4.transcode(d)  # the public call (allocates outputs, reads 32 bytes of counters back)
        # the expander's kernels alone, through the C ABI into preallocated buffers
        T_ = -(-k // 128)
        n_esc = a["esc"].numel() - 1
        scratch = torch.empty(4096 + n * k // 4, dtype=torch.uint8, device=dev)
        tmp_off, counters, row_cnt = torch.empty(n, dtype=torch.int32, device=dev), torch.empty(8, dtype=torch.int32, device=dev), torch.empty(n, dtype=torch.int32, device=dev)
        codes, flags, esc = torch.empty(n * T_ * 32, dtype=torch.int16, device=dev), torch.empty(n * T_, dtype=torch.uint8, device=dev), torch.empty(n_esc + 1, dtype=torch.uint8, device=dev)
        P = lambda t: ctypes.c_void_p(t.data_ptr())
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

        def expand_once():
            _native.call("cuda", "bn_rice_to_r4", P(d["meta"]), P(d["bits"]), d["bits"].numel(), P(d["roff"]), P(d["table"]), n, k, P(codes), P(flags), P(row_cnt), P(scratch), scratch.numel(), P(tmp_off), P(counters), stream)
            _native.call("cuda", "bn_r4_finish", P(row_cnt), P(scratch), P(tmp_off), n, P(row_cnt), P(esc), n_esc + 1, stream)

        expand_once()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 3
        ev0.record()
        for _ in range(reps):
            expand_once()
        ev1.record()
        torch.cuda.synchronize()
        expand_ms += ev0.elapsed_time(ev1) / reps
        want = o.pack_r4(u)
        as_np = lambda t, dt: t.cpu().numpy().view(dt)
        for got_t in ((a["codes"], a["flags"], a["esc"], a["row_esc"]), (codes, flags, esc, row_cnt)):
            if not (np.array_equal(as_np(got_t[0], np.uint16), want["codes"]) and np.array_equal(as_np(got_t[1], np.uint8), want["flags"]) and np.array_equal(as_np(got_t[2], np.uint8), want["esc"]) and np.array_equal(as_np(got_t[3], np.uint32), want["row_esc"])):
                raise SystemExit(f"bench: expander output of {name} differs from the oracle; refusing to report a number")
        del scratch, codes, flags, esc
        m0 = r4.R4Linear(a)  # adds the column-ordered escapes the batch-1 kernels walk (derived arrays, not in the reference's layout)
        want_cols, want_starts = o.esc_columns(want)
        if not (np.array_equal(as_np(a["esc_cols"], np.uint8), want_cols) and np.array_equal(as_np(a["col_esc"], np.uint16).reshape(n, 16), want_starts)):
            raise SystemExit(f"bench: column-ordered escapes of {name} differ from their definition restated in numpy; refusing to report a number")
        cols_tmp, starts_tmp = torch.empty_like(a["esc_cols"]), torch.empty_like(a["col_esc"])
        # (a short kernel: its calls are replayed from a CUDA graph so that the events time the
        # device work and not the host's launch rate)
        struct_a, cols_graph = ck.r4_struct(a), torch.cuda.CUDAGraph()
        with torch.cuda.graph(cols_graph):
            capture_stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
            for _ in range(reps):
                _native.call("cuda", "bn_r4_esc_columns", ctypes.byref(struct_a), n, k, P(cols_tmp), P(starts_tmp), capture_stream)
        cols_graph.replay()
        ev0.record()
        cols_graph.replay()
        ev1.record()
        torch.cuda.synchronize()
        columns_ms += ev0.elapsed_time(ev1) / reps
        del cols_graph
        del cols_tmp, starts_tmp
        if not np.array_equal(as_np(m0.dense().view(torch.int16), np.uint16).reshape(n, k), u):
            raise SystemExit(f"bench: dense decode of {name} differs from the source words; refusing to report a number")
        got_y = as_np(m0(ck.to_device(xs_host[k]).view(torch.bfloat16)).view(torch.int16), np.uint16)
        if not np.array_equal(got_y, o.c_r4_matvec(want, xs_host[k], n, k)):
            raise SystemExit(f"bench: GPU matvec of {name} differs from the oracle; refusing to report a number")
        parity["matrices"] += 1
        del want
        # algorithmic bytes of the expander: Rice arrays read + R4 arrays written (raw passes through)
        expand_bytes += sum(d[key].numel() * d[key].element_size() for key in ("meta", "bits", "roff", "table")) + sum(a[key].numel() * a[key].element_size() for key in ("codes", "flags", "esc", "row_esc"))
        bits_file += 8 * u.size + 8 * 256 + 8 * p["meta"].size + 32 * p["bits"].size + 32 * p["roff"].size
        bits_r4 += 8 * r4.r4_bytes(a)
        numel += u.size
        mods = [m0] + [r4.R4Linear({key: (v.clone() if torch.is_tensor(v) else v) for key, v in a.items()}) for _ in range(copies - 1)]
        layers.append((name, n, k, mods, r4.r4_bytes(a) + 2 * k + 2 * n))
        del d, p, u
    step_bytes = sum(l[4] for l in layers)
    note(f"{len(layers)} matrices packed, expanded and resident")
    xs = {k: ck.to_device(v).view(torch.bfloat16) for k, v in xs_host.items()}
    by_name = {name: (n, k, mods) for name, n, k, mods, _ in layers}
    groups = [g for g in ([nm for nm in grp if nm in by_name] for grp in GROUPS) if g]
    group_k = [by_name[g[0]][1] for g in groups]
    out_names = [nm for g in groups for nm in g]
    pushed = False
    exchanges = []
    if world > 1:
        # every rank's matrices are its row shard of a world-times taller layer: the public
        # sharded hook multiplies locally (one launch per group); the step's seven output slices
        # are then gathered in rank order with ONE collective (the step evaluates the four groups
        # on given inputs, so nothing needs a gathered vector before the step's end)
        from binade_b200.cuda.dist import RowShardedGroup, gather_all, make_exchange  # the library's peer-store all-gather, or NCCL

        stepper = [[RowShardedGroup([by_name[nm][2][c] for nm in g], [world * by_name[nm][0] for nm in g]) for g in groups] for c in range(copies)]
        exchanges = [make_exchange(max_bytes=2 * sum(by_name[nm][0] for nm in out_names) + 256) for c in range(copies)]
        pushed = exchanges[0] is not None

        xstream = torch.cuda.Stream(priority=-1)  # the exchange's own stream in the timed region; high priority: its small blocks are placed before the next product's

        def step(i: int, inputs=None, overlap: bool = False):
            # overlap: the exchange of this step runs on `xstream` while the current stream goes
            # on with the next step's products; the caller joins `xstream` before it ends
            inputs = inputs or xs
            slices = [y for grp, k in zip(stepper[i % copies], group_k) for y in grp(inputs[k], gather=False)]
            return gather_all(slices, exchange=exchanges[i % copies], stream=xstream if overlap else None)

    else:
        stepper = [[r4.R4LinearGroup([by_name[nm][2][c] for nm in g]) for g in groups] for c in range(copies)]

        xstream = None

        def step(i: int, inputs=None, overlap: bool = False):
            inputs = inputs or xs
            return [y for grp, k in zip(stepper[i % copies], group_k) for y in grp(inputs[k])]

    # ---- the step's own outputs: every group launch (and, with several GPUs, every gathered
    # vector on every rank) against the single-matrix products checked above
    for c in range(copies):
        outs = step(c)
        torch.cuda.synchronize()
        for nm, y in zip(out_names, outs):
            n, k, mods = by_name[nm]
            mine = mods[c](xs[k]).reshape(-1)
            if world == 1:
                ok = torch.equal(y.reshape(-1), mine)
            else:
                every = [torch.empty_like(mine) for _ in range(world)]
                dist.all_gather(every, mine)  # NCCL's gather of the slices checked above, on every rank
                ok = torch.equal(y.reshape(-1), torch.cat(every))
            if not ok:
                raise SystemExit(f"bench: output {nm} of the step differs from the checked single-matrix product (rank {rank}); refusing to report a number")
    parity["step_outputs"] = "grouped launches" + (f" and the gathered vectors on all {world} ranks" if world > 1 else "") + " bit-identical to the checked products"

    note("parity checked")
    # ---- timed region: W warm-up steps, then exactly K steps as replays of a CUDA graph that
    # holds GRAPH_ROUNDS steps per weight copy (plus a shorter graph for the remainder)
    for i in range(max(args.warmup, 3)):
        step(i)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())

    def capture(n_steps: int):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            step(0)
            side.synchronize()
            with torch.cuda.graph(g, stream=side):
                outs = [step(i, overlap=True) for i in range(n_steps)]
                if xstream is not None:
                    side.wait_stream(xstream)  # the graph ends when its last exchange has
        torch.cuda.synchronize()
        g.replay()  # untimed: graph upload
        torch.cuda.synchronize()
        return g, outs

    note("warm-up done")
    per_graph = copies * GRAPH_ROUNDS
    full, rem = divmod(args.steps, per_graph)
    g_full, outs_full = capture(per_graph) if full else (None, [])
    g_rem, outs_rem = capture(rem) if rem else (None, [])
    note("graphs captured")
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        ev0.record()
        for _ in range(full):
            g_full.replay()
        if g_rem:
            g_rem.replay()
        ev1.record()
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = ev0.elapsed_time(ev1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps
    for ex in exchanges:
        if ex is not None:
            ex.check()  # a wait that ran out on any rank voids the run
    # what the timed graphs left in their output buffers is what the checked eager step gives
    for outs in (outs_full, outs_rem):
        for c, got in enumerate(outs):
            want = step(c)
            torch.cuda.synchronize()
            if not all(torch.equal(a, b) for a, b in zip(got, want)):
                raise SystemExit(f"bench: the timed graph's outputs of step {c} differ from the checked step (rank {rank}); refusing to report a number")
    note(f"timed region done: {ms_per_step * 1e3:.1f} us per step")
    value = world * step_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- per shape: the matvec alone and cuBLAS BF16 GEMV on the pre-decoded weight, both
    # rotating the same copies inside a CUDA graph
    def graph_us(fn, iters=60):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            fn(0)
            side.synchronize()
            with torch.cuda.graph(g, stream=side):
                for i in range(iters):
                    fn(i)
        torch.cuda.synchronize()
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / iters

    per_shape = {}
    for name, n, k, mods, nbytes in layers if not args.quick else []:
        local = mods  # the rank's own modules (layers keeps them unwrapped)
        us = graph_us(lambda i: local[i % copies]._matvec(xs[k]))
        dense = [m.dense() for m in local]
        outs = [torch.empty(n, dtype=torch.bfloat16, device=dev) for _ in range(copies)]
        us_bf16 = graph_us(lambda i: torch.mv(dense[i % copies], xs[k], out=outs[i % copies]))
        per_shape[name] = {"us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1), "pct_of_8tbs": round(nbytes / us / 1e3 / NOMINAL_HBM_GBS * 100, 1), "bf16_gemv_us": round(us_bf16, 2), "speedup_vs_bf16": round(us_bf16 / us, 3)}
        del dense, outs

    # with several GPUs: every rank's own step without the exchange (the four local launches, same
    # rotation), so that the loss against one GPU can be split into the slowest GPU's pace and the
    # exchange's cost
    local_by_rank = None
    if world > 1:
        local_groups_all = [[r4.R4LinearGroup([by_name[nm][2][c] for nm in g]) for g in groups] for c in range(copies)]
        us_local = graph_us(lambda i: [grp(xs[k_]) for grp, k_ in zip(local_groups_all[i % copies], group_k)], iters=120)
        every = [torch.zeros(1, device=dev) for _ in range(world)]
        dist.all_gather(every, torch.tensor([us_local], device=dev))
        local_by_rank = [round(float(t.item()), 2) for t in every]
        del local_groups_all

    # the step's four launches, each alone (same rotation)
    per_launch = {}
    for gi, g in enumerate(groups if not args.quick else []):
        local_groups = [r4.R4LinearGroup([by_name[nm][2][c] for nm in g]) for c in range(copies)]
        us = graph_us(lambda i: local_groups[i % copies](xs[group_k[gi]]))
        nbytes = sum(l[4] for l in layers if l[0] in g) - 2 * group_k[gi] * (len(g) - 1)  # x is read once
        per_launch["+".join(g)] = {"us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1), "frac_of_measured_hbm": round(nbytes / us / 1e3 / measured_peaks()["hbm_gbs"], 3)}
    note("per-shape timings done")
    # ---- end to end through the public hook with host buffers: every step copies its inputs
    # from pinned host memory, runs the step and copies the seven outputs back to pinned host
    # memory, then synchronises. Measured twice: as eager calls, and with the same calls captured
    # once per weight copy in a CUDA graph that every step replays (how a serving loop runs a
    # fixed-shape step): the copies are nodes of the graph, so they are inside the timed region.
    k_list = sorted({k for _, _, k in SHAPES})
    h_x = {k: torch.from_numpy(xs_host[k].view(np.int16)).view(torch.bfloat16).pin_memory() for k in k_list}
    h_y = [torch.empty(n, dtype=torch.bfloat16).pin_memory() for _, n, _ in SHAPES]
    shape_index = {name: j for j, (name, _, _) in enumerate(SHAPES)}

    def e2e_body(i: int):
        dx = {k: h_x[k].to(dev, non_blocking=True) for k in k_list}
        for name, y in zip(out_names, step(i, dx)):  # the public hook (sharded groups with their collective when N > 1)
            j = shape_index[name]
            h_y[j].copy_(y.reshape(-1)[: SHAPES[j][1]], non_blocking=True)

    def timed(run, n_steps: int) -> float:
        for i in range(3):
            run(i)
        if world > 1:
            dist.barrier()
        ev0.record()
        for i in range(n_steps):
            run(i)
        ev1.record()
        torch.cuda.synchronize()
        t_ms = ev0.elapsed_time(ev1) / n_steps
        if world > 1:
            t = torch.tensor([t_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            t_ms = float(t.item())
        return t_ms

    def eager_step(i: int):
        e2e_body(i)
        torch.cuda.synchronize()

    e2e_steps = 3 if args.quick else min(args.steps, 200)
    e2e_eager_ms = timed(eager_step, e2e_steps)
    e2e_graphs = []
    for c in range(copies):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            e2e_body(c)
            side.synchronize()
            with torch.cuda.graph(g, stream=side):
                e2e_body(c)
        torch.cuda.synchronize()
        e2e_graphs.append(g)

    def graph_step(i: int):
        e2e_graphs[i % copies].replay()
        torch.cuda.synchronize()

    for j in range(len(h_y)):
        h_y[j].zero_()
    e2e_ms = timed(graph_step, e2e_steps)
    if rank == 0:  # what came back to the host is the checked product (the first slice is rank 0's)
        for name, (n, k, mods) in by_name.items():
            want = mods[(e2e_steps - 1) % copies](xs[k]).reshape(-1).cpu()
            if not torch.equal(h_y[shape_index[name]].view(torch.int16), want.view(torch.int16)):
                raise SystemExit(f"bench: the end-to-end step returned a wrong {name} to the host")
    e2e_val = world * step_bytes / (e2e_ms * 1e-3) / 1e9
    note("end-to-end leg done")

    # ---- whole-model decode: Llama-3.1-8B-shaped synthetic decoder, greedy, batch 1
    decode = None
    if not args.quick and not args.no_decode:
        from binade_b200.cuda.llama import Decoder, LlamaShape

        shape = LlamaShape()
        prompt = torch.randint(0, shape.vocab, (40,), device=dev, generator=torch.Generator(device=dev).manual_seed(1))
        decode = {"model": "Llama-3.1-8B-shaped synthetic decoder (32 layers, hidden 4096, FFN 14336, GQA 32/8 x 128, vocab 128256), N(0,0.02) BF16 weights, 40-token random prompt + 256 greedy tokens, one CUDA graph per token, linears row-sharded over the ranks"}
        for kind in ("r4", "bf16"):
            model = Decoder(shape, kind=kind, rank=rank, world=world)
            if kind == "r4":
                decode["checks"] = model.self_check()  # every R4 linear decodes to its source weight; first logits against fp32
            toks, secs = model.generate(prompt, 256)
            if world > 1:
                t = torch.tensor([secs], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                secs = float(t.item())
            decode[f"{kind}_tok_s"] = round(256 / secs, 1)
            decode[f"{kind}_weight_gb_per_token_per_gpu"] = round(model.linear_bytes() / 1e9, 3)
            del model
            torch.cuda.empty_cache()
        decode["r4_vs_bf16"] = round(decode["r4_tok_s"] / decode["bf16_tok_s"], 3)
        note(f"decode leg done: R4 {decode['r4_tok_s']} tok/s, BF16 {decode['bf16_tok_s']} tok/s")
    # ---- the other two configurations, single GPU only (no collective in them)
    prefill = moe_leg = config1 = None
    if world == 1 and args.prefill_rows:
        prefill = prefill_leg(torch, dev, graph_us, rows=tuple(int(v) for v in args.prefill_rows.split(",")))
    elif world == 1 and not args.quick:
        prefill, moe_leg = prefill_leg(torch, dev, graph_us), moe_path_leg(torch, dev, graph_us)
        note("prefill and MoE legs done")
        config1 = config1_leg(torch)
        note("configuration 1 done")
    elif world > 1 and not args.quick and 128 % world == 0:
        moe_leg = moe_parallel_leg(torch, dist, dev, rank, world)
        note("expert-parallel MoE leg done")
    if rank != 0:
        return None

    peaks = measured_peaks()
    launches = args.steps * len(groups)
    per_launch_bytes = step_bytes / len(groups)
    achieved = step_bytes / (ms_per_step * 1e-3) / 1e9
    result = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 weights (R4 coded), fp32 accumulate", "data": "synthetic",
        "config": {"workload": WORKLOAD, "copies_rotated": copies, "bytes_per_step": step_bytes, "launches_per_step": [" + ".join(g) for g in groups], "l2": f"each step streams {step_bytes / 1e6:.0f} MB of distinct weights (> 126 MB L2), {copies} copies rotated", "timing": f"CUDA-graph replays ({copies * GRAPH_ROUNDS} steps per graph, rotating the weight copies), CUDA events, max over ranks", "collective": ("peer-store all-gather kernel over NVLink (bn_push_gather)" if pushed else "NCCL all-gather") + " of the seven projection outputs, one per step, on a second stream: it overlaps the next step's products (steps are independent) and every graph ends after its last exchange" if world > 1 else "none"},
        "pct_of_nominal_8tbs": round(100 * value / world / NOMINAL_HBM_GBS, 2),
        "bits_per_weight": {"file_format2": round(bits_file / numel, 3), "r4_in_memory": round(bits_r4 / numel, 3)},
        "parity": parity,
        "shapes": per_shape,
        "launches": per_launch,
        "local_step_us_by_rank": local_by_rank,
        "speedup_vs_bf16_gemv_per_token": round(sum(v["bf16_gemv_us"] for v in per_shape.values()) / sum(v["us"] for v in per_shape.values()), 3) if per_shape else None,
        "expander": {"ms_per_layer": round(expand_ms, 3), "gbs": round(expand_bytes / expand_ms / 1e6, 1), "algorithmic_bytes": expand_bytes, "esc_columns_ms_per_layer": round(columns_ms, 3), "host_pack_s": round(host_pack_s, 2), "host_pack_cores": cpu_cores(), "gpu_pack_s": round(gpu_pack_s, 4)},
        "roofline": {"bound": "hbm", "kernel": f"r4_oct_kernel (all {len(groups)} launches of a step), averaged over them", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"], "bytes_per_launch": per_launch_bytes, "traffic": per_launch_bytes * NCU_TRAFFIC_RATIO, "traffic_source": "assumed, not measured in this run: DRAM read + write bytes of one ncu capture of the same kernel on the gate matrix, scaled to the average launch by its bytes"},
        "e2e": {"value": e2e_val, "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": sum(2 * k for k in k_list), "d2h_bytes_per_step": sum(2 * n for _, n, _ in SHAPES), "api": "R4LinearGroup.__call__ (RowShardedGroup + gather_all with several GPUs) on host-resident inputs, outputs copied back to pinned host memory; the calls of one step are captured once in a CUDA graph (copies included) and every step replays it and synchronises", "eager_ms_per_step": e2e_eager_ms, "eager_value": world * step_bytes / (e2e_eager_ms * 1e-3) / 1e9},
        "gpu_launches": launches,
        "decode": decode,
        "prefill_gate_15360x3840": prefill,
        "moe_128x(704x2816)": moe_leg,
        "config1_round_trip": config1,
        "clocks": clocks.summary(),
    }  # fmt: skip
    # ---- CPU baseline on a bounded sample (rank 0, single GPU runs only): the C restatement of
    # the same step on all host threads (the reference has no CPU matvec), and the numpy
    # restatement of its codec, which is what the reference itself runs on a CPU
    if world == 1 and not args.no_cpu and not args.quick:
        threads = o.set_threads(cpu_cores())
        mats = cpu_r4_layer(0)
        cpu_step(mats, xs_host)
        t0, n_rep = time.perf_counter(), 0
        while time.perf_counter() - t0 < 10.0 and n_rep < 200:
            cpu_step(mats, xs_host)
            n_rep += 1
        dt = (time.perf_counter() - t0) / n_rep
        result["cpu_baseline"] = {"value": sum(m[4] for m in mats) / dt / 1e9, "unit": UNIT, "cores": threads, "kind": "port", "sample": f"all 7 matvecs of the step, {n_rep} repetitions, C oracle with OpenMP over rows", "reference_codec_on_cpu": (config1 or {}).get("numpy_codec")}
    else:
        result["cpu_baseline"] = None
    return result


def same_order_rows(torch, x, w):
    """PyTorch fp32 reference of the documented summation order: x [M,K], w [N,K] bfloat16 ->
    [M,N] bfloat16. Lane l owns columns 128t + 4l + j; per lane sequential fp32 adds over t then
    j; lanes combine with strides 16, 8, 4, 2, 1; one rounding to BF16. (K % 128 == 0 here.)"""
    M, K = x.shape
    N, T = w.shape[0], K // 128
    out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    wf = w.float().view(N, T, 32, 4)
    for m0 in range(0, M, 64):  # bounded scratch: [64, N, 32] fp32 accumulators
        xf = x[m0 : m0 + 64].float().view(-1, 1, T, 32, 4)
        acc = torch.zeros((xf.shape[0], N, 32), dtype=torch.float32, device=x.device)
        for t in range(T):
            for j in range(4):
                acc += wf[None, :, t, :, j] * xf[:, :, t, :, j]  # the product of two BF16 values is exact in fp32
        for s in (16, 8, 4, 2, 1):
            acc = acc[..., :s] + acc[..., s : 2 * s]
        out[m0 : m0 + 64] = acc[..., 0].to(torch.bfloat16)
    return out


def prefill_leg(torch, dev, graph_us, rows=(2, 4, 8, 16, 32, 128, 256, 512, 2048)) -> dict:
    """Fused decode products for short prompts on the gate projection (15360 x 3840): M rows of
    N(0,1) inputs; up to FUSED_MAX_ROWS rows run the fused kernel in the documented order, up to
    MMA_MAX_ROWS the tensor-core decode GEMM (weights stream once in both), more rows rebuild the
    BF16 weight and call cuBLAS; against cuBLAS on the pre-decoded weight, and against the rebuild
    path where a fused kernel serves the row count. Every row count is also compared with the
    same-order fp32 reference: max_ulp is the largest deviation of an output in BF16 units in the
    last place (0 = bit-identical; the tensor-core paths sum in the hardware's order)."""
    from binade_b200.cuda import kernels as ck
    from binade_b200.cuda import r4

    n, k = 15360, 3840
    w = ck.to_device(synthetic_weight("gate", n, k)).view(torch.bfloat16)
    m = r4.R4Linear(r4.from_dense(w))
    if not torch.equal(m.dense().view(torch.int16), w.view(torch.int16)):
        raise SystemExit("bench: prefill weight does not decode to its source")
    out = {}
    for M in rows:
        x = torch.randn((M, k), device=dev, generator=torch.Generator(device=dev).manual_seed(M)).to(torch.bfloat16)
        us = graph_us(lambda i: m(x), iters=10)
        us_ref = graph_us(lambda i: torch.matmul(x, w.T), iters=10)
        path = "fused rows" if M <= r4.FUSED_MAX_ROWS else "tcgen05 decode GEMM" if M <= r4.MMA_MAX_ROWS * r4.MMA_MAX_PASSES else "rebuild + cuBLAS"
        got, ref = m(x), same_order_rows(torch, x, w)
        ulp = r4.ulp_distance(got, ref)
        # the same deviation measured against the size of what was summed: one BF16 ulp of
        # sum |w x| (an output that nearly cancels is many of its own ulps away after any reordering)
        scale = torch.exp2(torch.floor(torch.log2((x.float().abs() @ w.float().abs().T).clamp_min(1e-30))) - 7)
        rel = ((got.float() - ref.float()).abs() / scale).max().item()
        # and against cuBLAS itself on the pre-decoded weight: how many outputs carry the same bits
        same_as_cublas = float((got.view(torch.int16) == torch.matmul(x, w.T).view(torch.int16)).float().mean().item())
        out[str(M)] = {"us": round(us, 1), "cublas_bf16_us": round(us_ref, 1), "vs_cublas": round(us_ref / us, 3), "path": path, "outputs_identical_to_cublas": round(same_as_cublas, 6), "max_ulp": int(ulp.max().item()), "outputs_not_identical": round(float((ulp > 0).float().mean().item()), 5), "outputs_beyond_1_ulp": round(float((ulp > 1).float().mean().item()), 6), "max_err_in_ulps_of_sum_abs": round(rel, 4)}
        if M <= r4.MMA_MAX_ROWS * r4.MMA_MAX_PASSES:
            out[str(M)]["rebuild_us"] = round(graph_us(lambda i: x @ m.dense().reshape(n, k).T, iters=10), 1)
    # the order of cuBLAS: the split-K count with which the tensor-core kernel gives the bits of
    # torch's BF16 matmul on the decoded weight, for this matrix and for the down projection
    # (long K: cuBLAS splits K for few rows), each checked on fresh inputs
    if any(M <= r4.MMA_MAX_ROWS for M in rows):
        mirror = {}
        for name, nn_, kk_ in (("gate_15360x3840", n, k), ("down_3840x15360", 3840, 15360)):
            wd = w if (nn_, kk_) == (n, k) else ck.to_device(synthetic_weight("down", nn_, kk_)).view(torch.bfloat16)
            md = m if wd is w else r4.R4Linear(r4.from_dense(wd))
            plan = md.mirror_cublas(rows=(8, 16, 32, 128))
            same = {}
            for M, split in plan.items():
                xm = torch.randn((M, kk_), device=dev, generator=torch.Generator(device=dev).manual_seed(1000 + M)).to(torch.bfloat16)
                same[str(M)] = {"split_k": split, "outputs_identical_to_cublas": round(float((md.mma_rows(xm).view(torch.int16) == (xm @ wd.T).view(torch.int16)).float().mean().item()), 6)}
            mirror[name] = same
        out["cublas_order"] = mirror
    return out


def moe_path_leg(torch, dev, graph_us) -> dict:
    """Expert path of a 26B-A4B-style layer: 128 experts, top-8 of uniform random logits, hidden
    2816, expert FFN 704, token batches 1/8/64; fused gate+up gather, SwiGLU, down gather; a
    batch with more slots than twice the experts is grouped by expert (weights read once).
    Checked at this size: both weight stacks decode to their sources, and for every batch the
    gate/up gather and the down gather equal the CPU oracle's gathers bit for bit (the down
    gather on the activations the GPU produced), and the layer's output equals their chain."""
    from binade_b200.cuda import moe, r4
    from oracle import oracle as o

    E, n, D = 128, 704, 2816
    g = torch.Generator(device=dev).manual_seed(5)
    gu = (torch.randn((E, 2 * n, D), device=dev, generator=g) * 0.02).to(torch.bfloat16)
    dn = (torch.randn((E, D, n), device=dev, generator=g) * 0.02).to(torch.bfloat16)
    layer = moe.R4SwitchGLU(r4.R4Linear(r4.from_dense(gu)), r4.R4Linear(r4.from_dense(dn)))
    if not (torch.equal(layer._gu.dense().view(torch.int16), gu.view(torch.int16)) and torch.equal(layer._down.dense().view(torch.int16), dn.view(torch.int16))):
        raise SystemExit("bench: MoE expert weights do not decode to their sources")
    per_expert = (r4.r4_bytes(layer._gu._a) + r4.r4_bytes(layer._down._a)) / E
    del gu, dn
    host = lambda a: {key: a[key].cpu().numpy().view({"codes": np.uint16, "row_esc": np.uint32}.get(key, np.uint8)) for key in ("raw", "codes", "flags", "esc", "table", "row_esc")}
    a_gu, a_dn = host(layer._gu._a), host(layer._down._a)
    u16 = lambda t: t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    out = {}
    for B in (1, 8, 64):
        x = torch.randn((B, D), device=dev, generator=g).to(torch.bfloat16)
        idx = torch.topk(torch.softmax(torch.rand((B, E), device=dev, generator=g), dim=-1), 8, dim=-1).indices
        y = layer(x, idx)
        ei = idx.reshape(-1).to(torch.int32)
        xi = torch.arange(ei.numel(), dtype=torch.int32, device=dev) // 8
        gate, up = layer._gu._gather(x, xi, ei, 2 * n, 2 * n, split=n)
        ei_np, xi_np = ei.cpu().numpy().astype(np.uint32), xi.cpu().numpy().astype(np.uint32)
        want_gu = o.c_r4_gather(a_gu, u16(x), xi_np, ei_np, 2 * n, D, 2 * n)
        h = moe.swiglu(up, gate)
        rows = np.arange(ei.numel(), dtype=np.uint32)
        want_dn = o.c_r4_gather(a_dn, u16(h), rows, ei_np, D, n, D)
        if not (np.array_equal(u16(gate), want_gu[:, :n]) and np.array_equal(u16(up), want_gu[:, n:]) and np.array_equal(u16(y.reshape(-1, D)), want_dn)):
            raise SystemExit(f"bench: MoE expert path differs from the oracle at {B} tokens")
        us = graph_us(lambda i: layer(x, idx), iters=10)
        active = int(torch.unique(idx).numel())
        grouped = B * 8 >= layer.GROUP_MIN_SLOTS * E  # slots grouped by expert: every active expert is read once
        out[str(B)] = {"us": round(us, 1), "slots": B * 8, "active_experts": active, "path": "grouped by expert" if grouped else "slot by slot", "gbs_of_slot_bytes": round(B * 8 * per_expert / us / 1e3, 1), "gbs_of_distinct_expert_bytes": round(active * per_expert / us / 1e3, 1), "checked": "gathers and layer output bit-identical to the oracle"}
    return out


def moe_parallel_leg(torch, dist, dev, rank: int, world: int) -> dict:
    """The same expert layer with its 128 experts and the token batch split over the ranks:
    ExpertParallelGLU (all-to-all dispatch of the slots' input rows to the ranks owning their
    experts, the local expert path, all-to-all combine). Every rank checks its tokens' outputs
    bit for bit against the whole layer on its own GPU, then the forward is timed eagerly with
    CUDA events (max over ranks). Batches of 1 / 8 / 64 tokens in all; a rank without a real
    token brings a padding token."""
    from binade_b200.cuda import moe, r4

    E, n, D, k = 128, 704, 2816, 8
    per = E // world
    g = torch.Generator(device=dev).manual_seed(5)
    gu = (torch.randn((E, 2 * n, D), device=dev, generator=g) * 0.02).to(torch.bfloat16)
    dn = (torch.randn((E, D, n), device=dev, generator=g) * 0.02).to(torch.bfloat16)
    whole = moe.R4SwitchGLU(r4.R4Linear(r4.from_dense(gu)), r4.R4Linear(r4.from_dense(dn)))
    local = moe.R4SwitchGLU(r4.R4Linear(r4.from_dense(gu[rank * per : (rank + 1) * per].contiguous())), r4.R4Linear(r4.from_dense(dn[rank * per : (rank + 1) * per].contiguous())))
    del gu, dn
    ep = moe.ExpertParallelGLU(local.slots, E, D, rank, world)
    out = {}
    for B in (1, 8, 64):
        each = -(-B // world)
        x = torch.randn((each * world, D), device=dev, generator=g).to(torch.bfloat16)
        idx = torch.topk(torch.softmax(torch.rand((each * world, E), device=dev, generator=g), dim=-1), k, dim=-1).indices
        idx[B:] = -1  # padding tokens
        mine = slice(rank * each, (rank + 1) * each)
        y = ep(x[mine], idx[mine])
        want = whole(x[mine], idx[mine].clamp(min=0))
        want[idx[mine] < 0] = 0
        if not torch.equal(y.view(torch.int16), want.view(torch.int16)):
            raise SystemExit(f"bench: expert-parallel output differs from the single-GPU layer at {B} tokens (rank {rank})")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(3):
            ep(x[mine], idx[mine])
        dist.barrier()
        e0.record()
        for _ in range(20):
            ep(x[mine], idx[mine])
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / 20], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e0.record()
        for _ in range(20):
            whole(x[:B], idx[:B])
        e1.record()
        torch.cuda.synchronize()
        single_us = e0.elapsed_time(e1) * 1e3 / 20
        # the same forward captured once in a CUDA graph (fixed shapes, no host synchronisation
        # inside, the all-to-alls are nodes of the graph) and replayed; the ranks agree that all
        # of them captured it before any of them replays
        graph_us, captured, gph, yg = None, 1, None, None
        try:
            gph = torch.cuda.CUDAGraph()
            cap = torch.cuda.Stream()
            cap.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(cap):
                with torch.cuda.graph(gph, stream=cap):
                    yg = ep(x[mine], idx[mine])
            torch.cuda.synchronize()
        except Exception as e:  # noqa: BLE001 - reported in the JSON line, the eager number stands
            captured, graph_us = 0, f"not captured: {type(e).__name__}"
        flag = torch.tensor([captured], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()):
            gph.replay()
            torch.cuda.synchronize()
            if not torch.equal(yg.view(torch.int16), want.view(torch.int16)):
                raise SystemExit(f"bench: the captured expert-parallel forward differs from the single-GPU layer at {B} tokens (rank {rank})")
            dist.barrier()
            e0.record()
            for _ in range(20):
                gph.replay()
            e1.record()
            torch.cuda.synchronize()
            tg = torch.tensor([e0.elapsed_time(e1) * 1e3 / 20], device=dev)
            dist.all_reduce(tg, op=dist.ReduceOp.MAX)
            graph_us = round(float(tg.item()), 1)
        elif captured:
            graph_us = "not captured on another rank"
        out[str(B)] = {"us": round(float(t.item()), 1), "graph_replay_us": graph_us, "single_gpu_layer_us_eager": round(single_us, 1), "tokens_per_rank": each, "experts_per_rank": per, "checked": "bit-identical to the single-GPU layer on every rank", "timing": "us: eager launches (torch glue + 2 all-to-all + 2 gather kernels); graph_replay_us: the forward captured once and replayed; CUDA events, max over ranks"}
    return out


def config1_leg(torch) -> dict:
    """Configuration 1 as stated: one BF16 tensor 2048 x 2048 from seed 0, N(0, 0.02), 0.1 % of
    entries scaled x64, 0.01 % set to +-0 or a subnormal; pack (format 2) and unpack must give
    the tensor back bit for bit; bits per weight of the file arrays. The same tensor times the
    numpy restatement of the reference's codec (its encoder and decoder are numpy loops over
    planes, binade/rice.py:76-173) on one host core, next to the package's C++ encoder and the
    GPU decoder."""
    from binade_b200 import pack, unpack
    from oracle import oracle as o

    g = torch.Generator().manual_seed(0)
    w = torch.randn((2048, 2048), generator=g) * 0.02
    w = torch.where(torch.rand((2048, 2048), generator=g) < 1e-3, w * 64, w)
    u = w.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16).copy()
    special = torch.rand((2048, 2048), generator=g).numpy() < 1e-4
    kinds = np.array([0x0000, 0x8000, 0x0001, 0x8001, 0x007F, 0x0040], np.uint16)  # +-0 and subnormals
    u[special] = kinds[torch.randint(0, len(kinds), (int(special.sum()),), generator=g).numpy()]
    t0 = time.perf_counter()
    p = pack.pack(u)
    t_pack = time.perf_counter() - t0
    t0 = time.perf_counter()
    back = unpack.unpack(p)
    torch.cuda.synchronize()
    t_unpack = time.perf_counter() - t0
    if not np.array_equal(back, u):
        raise SystemExit("bench: unpack(pack(w)) differs from w on configuration 1")
    # the reference's numpy codec, restated: split, rank table, encode, decode, join
    t0 = time.perf_counter()
    raw, exps = o.np_split(u)
    table, rank = o.np_rank_table(np.bincount(exps.reshape(-1), minlength=256))
    meta, words_, roff = o.np_rice_encode_ranks(rank[exps])
    t_enc = time.perf_counter() - t0
    t0 = time.perf_counter()
    ranks, _ = o.np_rice_decode_ranks(meta, words_, roff, 2048)
    again = o.np_join(raw, table[ranks[:, :2048]])
    t_dec = time.perf_counter() - t0
    if not (np.array_equal(again, u) and np.array_equal(np.asarray(p["bits"]).reshape(-1), np.asarray(words_).reshape(-1))):
        raise SystemExit("bench: the numpy codec and the package's packer disagree on configuration 1")
    return {
        "tensor": "2048 x 2048 BF16, seed 0, N(0,0.02), 0.1 % x64, 0.01 % +-0 / subnormal", "round_trip": "bit-identical (C++ pack, GPU unpack; numpy encode / decode)",
        "bits_per_weight": round(pack.bits_per_weight(p), 3), "escaped_or_special_entries": int(special.sum()),
        "numpy_codec": {"encode_s": round(t_enc, 2), "decode_s": round(t_dec, 2), "encode_mweights_s": round(u.size / t_enc / 1e6, 2), "decode_mweights_s": round(u.size / t_dec / 1e6, 2), "cores_used": 1, "cpu_count": os.cpu_count(), "affinity": cpu_cores()},
        "this_package": {"pack_s": round(t_pack, 3), "pack_cores": cpu_cores(), "gpu_unpack_s_with_copies": round(t_unpack, 3)},
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--copies", type=int, default=3, help="weight copies rotated between steps")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-decode", action="store_true", help="skip the whole-model decode leg")
    ap.add_argument("--shapes", default="", help="comma list of matrices to keep (default: all seven); for small profiling runs")
    ap.add_argument("--prefill-rows", default="", help="comma list of input row counts: run the prefill leg on just these (with --quick, for profiling runs)")
    ap.add_argument("--quick", action="store_true", help="timed region only: skip the per-shape, end-to-end and CPU legs")
    args = ap.parse_args()
    if args.shapes:
        keep = set(args.shapes.split(","))
        SHAPES[:] = [sh for sh in SHAPES if sh[0] in keep]
    if args.impl == "reference":
        if int(os.environ.get("RANK", 0)) != 0:
            return
        print(json.dumps(run_reference(args)))
        return
    out = run_ours(args)
    if out is not None:
        print(json.dumps(out), flush=True)
    if int(os.environ.get("WORLD_SIZE", 1)) > 1:
        # Leave together and at once: tearing the NCCL communicator down while captured graphs
        # still hold its kernels has been seen to block; the result line is already out.
        import torch
        import torch.distributed as dist

        torch.cuda.synchronize()
        dist.barrier()
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
