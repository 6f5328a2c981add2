"""A bounded wait that is seen to run out, without faulting or hanging the GPU: the peer-store
exchange is called as rank 0 of two, with a second local buffer standing in for the peer whose
flag nothing ever raises. The kernel must return, the device status must say so, a reset must
clear it, and the next normal call must work."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _status() -> int:
    from binade_b200 import _native

    st = ctypes.c_int(-1)
    _native.call("cuda", "bn_device_status", ctypes.byref(st))
    return st.value


def _push(local, peers, area, out, rank, world, counter, entry="bn_push_gather"):
    from binade_b200 import _native

    ptrs = (ctypes.c_void_p * 1)(local.data_ptr())
    lens = (ctypes.c_uint64 * 1)(local.numel() * local.element_size())
    addr = (ctypes.c_uint64 * world)(*[p.data_ptr() for p in peers])
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _native.call("cuda", entry, ctypes.cast(ptrs, ctypes.c_void_p), ctypes.cast(lens, ctypes.c_void_p), 1, ctypes.cast(addr, ctypes.c_void_p), area, ctypes.c_void_p(out.data_ptr()), rank, world, ctypes.c_void_p(counter.data_ptr()), stream)


def test_absent_peer_ends_in_a_status_not_a_hang():
    from binade_b200 import _native

    assert _status() == 0
    area = 1024
    mine = torch.zeros(256 + 2 * area, dtype=torch.uint8, device="cuda")
    absent = torch.zeros_like(mine)  # the "peer": its rank never runs, so it never raises its flag in `mine`
    out = torch.zeros(area, dtype=torch.uint8, device="cuda")
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    piece = torch.arange(64, dtype=torch.uint8, device="cuda")
    _native.call("cuda", "bn_set_wait_limit_ns", 30_000_000)  # 30 ms instead of two seconds
    try:
        _push(piece, [mine, absent], area, out, 0, 2, counter)
        torch.cuda.synchronize()  # the kernel returned: no hang
        assert _status() & 0xFF0000, "the exchange kernel must report the wait it gave up"
        assert not out.any()  # nothing was copied to the output
        # the store side did run: the slice sits in both buffers' first area (exchange number 1 uses area 1)
        assert torch.equal(absent[256 + area : 256 + area + 64], piece)
    finally:
        _native.call("cuda", "bn_set_wait_limit_ns", 0)
        _native.call("cuda", "bn_device_status_reset")
    assert _status() == 0
    # the context is intact: a one-rank exchange completes and copies its slice out
    solo = torch.zeros(256 + 2 * area, dtype=torch.uint8, device="cuda")
    counter.zero_()
    _push(piece, [solo], area, out, 0, 1, counter)
    torch.cuda.synchronize()
    assert torch.equal(out[:64], piece) and _status() == 0


def test_three_kernel_exchange_gives_up_and_recovers_too():
    """The form for a stream of its own (stores, a one-warp wait, copy-out as three launches):
    the absent peer ends in the same status with nothing copied out and the call number still
    advanced, so that the next call, of either form, on the same buffers works."""
    from binade_b200 import _native

    area = 1024
    mine = torch.zeros(256 + 2 * area, dtype=torch.uint8, device="cuda")
    absent = torch.zeros_like(mine)
    out = torch.zeros(area, dtype=torch.uint8, device="cuda")
    counter = torch.zeros(4, dtype=torch.int32, device="cuda")
    piece = torch.arange(64, dtype=torch.uint8, device="cuda")
    _native.call("cuda", "bn_set_wait_limit_ns", 30_000_000)
    try:
        _push(piece, [mine, absent], area, out, 0, 2, counter, "bn_push_gather_beside")
        torch.cuda.synchronize()
        assert _status() & 0xFF0000 and not out.any()
        assert torch.equal(absent[256 + area : 256 + area + 64], piece)
        assert counter.tolist() == [1, 0, 0, 0]  # call 1 is over, tickets back at zero, the wait failed
    finally:
        _native.call("cuda", "bn_set_wait_limit_ns", 0)
        _native.call("cuda", "bn_device_status_reset")
    solo = torch.zeros(256 + 2 * area, dtype=torch.uint8, device="cuda")
    for call, entry in enumerate(("bn_push_gather_beside", "bn_push_gather", "bn_push_gather_beside"), 2):
        out.zero_()
        _push(piece + call, [solo], area, out, 0, 1, counter, entry)
        torch.cuda.synchronize()
        assert torch.equal(out[:64], piece + call) and counter[0].item() == call and _status() == 0
