"""The expander entry point that allocates nothing (bn_rice_to_r4_static), through the C ABI.

It exists for callers that cannot allocate device memory while loading weights (a plugin under
a framework whose allocator owns the device, a loader beside a stream capture, a fixed-budget
service). Its outputs must equal those of the two-step expander that takes caller scratch, call
after call: the fixed scratch array keeps whatever the previous call left in it."""

import ctypes

import numpy as np
import pytest
import torch

from test_gpu_parity import dev, packed_arrays, weights

pytestmark = pytest.mark.gpu


def expand_static(p: dict, esc_cap: int):
    from binade_b200 import _native

    R, K = p["raw"].reshape(-1, p["shape"][-1]).shape
    T = -(-K // 128)
    d = {k: dev(p[k]) for k in ("meta", "bits", "roff", "table")}
    codes = torch.full((R * T * 32,), -1, dtype=torch.int16, device="cuda")
    flags = torch.full((R * T,), 255, dtype=torch.uint8, device="cuda")
    row_esc = torch.full((R,), -1, dtype=torch.int32, device="cuda")
    esc = torch.full((esc_cap,), 255, dtype=torch.uint8, device="cuda")
    info = torch.full((4,), -1, dtype=torch.int32, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    _native.call("cuda", "bn_rice_to_r4_static", ptr(d["meta"]), ptr(d["bits"]), d["bits"].numel(), ptr(d["roff"]), ptr(d["table"]), R, K, ptr(codes), ptr(flags), ptr(row_esc), ptr(esc), esc_cap, ptr(info), stream)
    torch.cuda.synchronize()
    return codes, flags, row_esc, esc, info.cpu().numpy().view(np.uint32)


def check(u: np.ndarray):
    from binade_b200.cuda import r4

    p = packed_arrays(u)
    want = r4.transcode(p)  # the existing entry points: bn_rice_to_r4 + bn_r4_finish
    n = want["esc"].numel() - 1
    codes, flags, row_esc, esc, info = expand_static(p, n + 1 + 64)
    assert info.tolist() == [n, 0, 0, 0]
    assert torch.equal(codes, want["codes"]) and torch.equal(flags, want["flags"]) and torch.equal(row_esc, want["row_esc"])
    assert torch.equal(esc[: n + 1], want["esc"])
    # and directly against the CPU oracle's arrays (the reference's transcode, restated)
    from oracle import oracle as o

    ref = o.pack_r4(u.reshape(-1, u.shape[-1]))
    assert np.array_equal(codes.cpu().numpy().view(np.uint16), ref["codes"]) and np.array_equal(flags.cpu().numpy(), ref["flags"])
    assert np.array_equal(row_esc.cpu().numpy().view(np.uint32), ref["row_esc"]) and np.array_equal(esc[: n + 1].cpu().numpy(), ref["esc"])


def test_static_expander_matches_two_calls_in_a_row():
    rng = np.random.default_rng(11)
    first = weights(rng, (300, 3840))
    check(first)
    # a second, different matrix right after: nothing of the first call may leak through the scratch
    check(rng.integers(0, 1 << 16, size=(64, 1024), dtype=np.uint16))  # nearly every weight escapes
    check(first)
    check(weights(rng, (48, 100), escapes=False))


def test_static_expander_limits_and_errors():
    from binade_b200 import _native

    u = weights(np.random.default_rng(12), (8, 256))
    p = packed_arrays(u)
    # esc too small: reported on the device, nothing written past the capacity
    codes, flags, row_esc, esc, info = expand_static(p, 3)
    assert info[2] == 1 and info[0] > 2 and esc[2].item() == 0
    # a corrupt stream: the first bad row is reported
    bad = dict(p, bits=p["bits"][:-1])
    _, _, _, _, info = expand_static(bad, 4096)
    assert info[1] == 1  # R - (R - 1): the last row
    # beyond the fixed scratch: refused on the host before any launch
    z = torch.zeros(8, dtype=torch.int32, device="cuda")
    ptr = ctypes.c_void_p(z.data_ptr())
    for R, K in ((65537, 4), (8192, 4096)):
        with pytest.raises(_native.NativeError, match="at most 65536 rows"):
            _native.call("cuda", "bn_rice_to_r4_static", ptr, ptr, 0, ptr, ptr, R, K, ptr, ptr, ptr, ptr, 8, ptr, None)
