"""Packed model on disk -> R4 arrays on the device, with the file reads overlapped.

The reference reads every file array with a blocking `np.fromfile` (binade/st.py:85-94), then
moves it to the device, then transcodes it, one tensor after another. Here a reader thread reads
the next tensor's arrays straight into pinned host buffers (`readinto`, no intermediate copy)
while the current tensor's arrays are copied to the device from the other set of pinned buffers
and expanded there: the disk, the copy engine and the SMs work at the same time.

    for name, a in stream_r4(packed_dir):        # a: the dict r4.transcode returns
        modules[name] = r4.R4Linear(a)
"""

from __future__ import annotations

import queue
import threading

import torch

from .. import st
from ..unpack import PackedModel
from . import r4

PARTS2 = ("raw", "table", "meta", "bits", "roff")  # format 2 (Rice)
PARTS1 = ("raw", "table", "meta", "idx", "esc")  # format 1 (fixed-width codes)


class _Slot:
    """One set of pinned staging buffers, one per file array, grown on demand and reused."""

    def __init__(self):
        self.buf: dict = {}

    def view(self, part: str, nbytes: int) -> torch.Tensor:
        t = self.buf.get(part)
        if t is None or t.numel() < nbytes:
            t = self.buf[part] = torch.empty(max(nbytes, 1), dtype=torch.uint8, pin_memory=True)
        return t[:nbytes]


def _read_into(info: st.TensorInfo, out: torch.Tensor) -> None:
    """The tensor's bytes from its safetensors file into `out` (pinned uint8), no copy between."""
    target = memoryview(out.numpy())
    with open(info.file, "rb", buffering=0) as f:
        f.seek(info.offset)
        got = 0
        while got < len(target):
            n = f.readinto(target[got:])
            if not n:
                raise OSError(f"{info.file}: {info.name} ends after {got} of {len(target)} bytes")
            got += n


def stream_r4(packed, names=None, slots: int = 2):
    """Yield (name, R4 arrays) for the packed weights of a model directory (or PackedModel), in
    `names` order (default: file order), reading ahead by `slots - 1` tensors. The arrays equal
    `r4.transcode` of the same file arrays. Raises what `transcode` raises on a bad stream; a read
    error of the reader thread is raised here at the tensor it belongs to."""
    pm = packed if isinstance(packed, PackedModel) else PackedModel(packed)
    names = list(pm.packed if names is None else names)
    free, ready = queue.Queue(), queue.Queue()
    for _ in range(max(slots, 1)):
        free.put(_Slot())
    stop = threading.Event()

    def parts_of(name):
        return PARTS2 if f"{name}.bits" in pm.infos else PARTS1

    def reader():
        for name in names:
            slot = free.get()
            if stop.is_set():
                return
            try:
                views = {}
                for part in parts_of(name):
                    info = pm.infos[f"{name}.{part}"]
                    views[part] = (slot.view(part, info.nbytes), info)
                    _read_into(info, views[part][0])
                ready.put((name, slot, views, None))
            except Exception as e:  # noqa: BLE001 - handed to the consumer, which raises it in order
                ready.put((name, slot, None, e))
                return

    thread = threading.Thread(target=reader, name="binade-b200-reader", daemon=True)
    thread.start()
    copy_stream = torch.cuda.Stream()
    try:
        for _ in names:
            name, slot, views, err = ready.get()
            if err is not None:
                raise err
            w = {}
            with torch.cuda.stream(copy_stream):
                for part, (host, info) in views.items():
                    dt = {"U8": torch.uint8, "U16": torch.int16, "U32": torch.int32}[info.dtype]
                    d = host.to("cuda", non_blocking=True).view(dt)
                    w[part] = d.reshape(info.shape) if part == "raw" else d
                copied = torch.cuda.Event()
                copied.record(copy_stream)
            torch.cuda.current_stream().wait_stream(copy_stream)
            for d in w.values():
                d.record_stream(torch.cuda.current_stream())
            a = r4.transcode(w)
            copied.synchronize()
            free.put(slot)  # the copies have left the pinned buffers: the reader may overwrite them
            yield name, a
    finally:
        stop.set()
        free.put(_Slot())  # wakes a reader waiting for a slot so that it can leave
