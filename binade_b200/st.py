"""safetensors files as byte ranges: header parsing, row-range reads, a streaming writer.

BF16 tensors are handled as uint16 bit patterns (numpy has no bfloat16). A file is
  8 bytes little-endian header length | JSON header (may be space padded) | tensor data
and each header entry gives dtype, shape and [begin, end) offsets into the data section.
Same role as the reference's binade/st.py; the writer reserves header room up front exactly as
the reference does, so packed files come out byte-identical.
"""

from __future__ import annotations

import json
import math
import re
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np

NP_DTYPE = {
    "BOOL": np.bool_, "U8": np.uint8, "I8": np.int8, "U16": np.uint16, "I16": np.int16,
    "F16": np.float16, "BF16": np.uint16, "U32": np.uint32, "I32": np.int32, "F32": np.float32,
    "U64": np.uint64, "I64": np.int64, "F64": np.float64,
}  # fmt: skip
ST_DTYPE = {np.dtype(np.uint8): "U8", np.dtype(np.uint16): "U16", np.dtype(np.uint32): "U32", np.dtype(np.float32): "F32"}
INDEX = "model.safetensors.index.json"


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: tuple
    file: Path
    offset: int  # absolute byte offset of the tensor's data in `file`
    nbytes: int

    @property
    def numel(self) -> int:
        return math.prod(self.shape)

    @property
    def rows(self) -> int:
        """Rows of the 2-D view [prod(shape[:-1]), shape[-1]]; tiles never cross a row."""
        return math.prod(self.shape[:-1]) if self.shape else 1


def read_header(path):
    """(header dict, offset of the data section)."""
    with open(path, "rb") as f:
        (size,) = struct.unpack("<Q", f.read(8))
        return json.loads(f.read(size)), 8 + size


def shard_files(model_dir):
    """The model's safetensors files: those the index names, else every *.safetensors."""
    model_dir = Path(model_dir)
    if (model_dir / INDEX).exists():
        names = set(json.loads((model_dir / INDEX).read_text())["weight_map"].values())
    else:
        names = {p.name for p in model_dir.glob("*.safetensors")}
    if not names:
        raise FileNotFoundError(f"no safetensors files in {model_dir}")
    return [model_dir / n for n in sorted(names)]


def list_tensors(model_dir):
    """Every tensor of a model directory, ordered by file then position in the file."""
    infos = []
    for path in shard_files(model_dir):
        header, base = read_header(path)
        for name, entry in header.items():
            if name != "__metadata__":
                begin, end = entry["data_offsets"]
                infos.append(TensorInfo(name, entry["dtype"], tuple(entry["shape"]), path, base + begin, end - begin))
    infos.sort(key=lambda t: (str(t.file), t.offset))
    return infos


def read(info: TensorInfo, rows=None) -> np.ndarray:
    """A whole tensor, or rows [r0, r1) of its 2-D view."""
    dt = np.dtype(NP_DTYPE[info.dtype])
    if rows is None:
        return np.fromfile(info.file, dtype=dt, count=info.numel, offset=info.offset).reshape(info.shape)
    r0, r1 = rows
    width = info.shape[-1]
    data = np.fromfile(info.file, dtype=dt, count=(r1 - r0) * width, offset=info.offset + r0 * width * dt.itemsize)
    return data.reshape(r1 - r0, width)


_HF_SNAPSHOT = re.compile(r"models--(?P<org>[^/]+?)--(?P<name>[^/]+)/snapshots/(?P<rev>[0-9a-f]{40})")


def resolve(model: str, revision: str | None = None) -> Path:
    """A local directory, or a Hugging Face repo id already in the local cache (no download)."""
    local = Path(model).expanduser()
    if local.is_dir():
        return local.resolve()
    try:
        from huggingface_hub import scan_cache_dir
    except ImportError as e:
        raise FileNotFoundError(f"{model}: not a directory, and huggingface_hub is not installed") from e
    hits = [
        rev
        for repo in scan_cache_dir().repos
        if repo.repo_id == model and repo.repo_type == "model"
        for rev in repo.revisions
        if revision is None or rev.commit_hash.startswith(revision) or revision in rev.refs
    ]
    if len(hits) != 1:
        raise FileNotFoundError(f"{model}: {len(hits)} matching cached snapshots; download it or pass --revision")
    return Path(hits[0].snapshot_path)


def fetch(model: str, revision: str | None = None) -> Path:
    """Like resolve; an uncached `org/name` repo id is downloaded when huggingface_hub can."""
    try:
        return resolve(model, revision)
    except FileNotFoundError:
        if Path(model).expanduser().exists() or model.count("/") != 1:
            raise
    from huggingface_hub import snapshot_download

    return Path(snapshot_download(model, revision=revision))


def provenance(model_dir) -> dict:
    """Where a model came from: its path, plus repo id and revision for an HF cache snapshot."""
    m = _HF_SNAPSHOT.search(str(model_dir))
    out = {"path": str(model_dir)}
    if m:
        out.update(repo_id=f"{m['org']}/{m['name']}", revision=m["rev"])
    return out


class Writer:
    """Streaming safetensors writer: tensors are appended back to back, the header is written
    last into `reserve` bytes kept free at the start (space padded, which the format allows)."""

    def __init__(self, path, reserve: int, metadata: dict | None = None):
        self.path = Path(path)
        self.reserve = -(-reserve // 8) * 8
        self.metadata = dict(metadata or {})
        self.entries: dict = {}
        self.pos = 0
        self._current = None
        self.f = open(self.path, "wb")
        self.f.write(bytes(8 + self.reserve))

    def begin(self, name: str, dtype: str, shape) -> None:
        if self._current is not None or name in self.entries:
            raise ValueError(f"{name}: tensor already open or written")
        self._current = (name, dtype, [int(s) for s in shape], self.pos)

    def write(self, data: np.ndarray) -> None:
        blob = np.ascontiguousarray(data).tobytes()
        self.f.write(blob)
        self.pos += len(blob)

    def end(self) -> None:
        name, dtype, shape, start = self._current
        want = math.prod(shape) * np.dtype(NP_DTYPE[dtype]).itemsize
        if self.pos - start != want:
            raise ValueError(f"{name}: wrote {self.pos - start} bytes, shape {shape} {dtype} needs {want}")
        self.entries[name] = {"dtype": dtype, "shape": shape, "data_offsets": [start, self.pos]}
        self._current = None

    def add(self, name: str, a: np.ndarray, dtype: str | None = None) -> None:
        self.begin(name, dtype or ST_DTYPE[a.dtype], a.shape)
        self.write(a)
        self.end()

    def close(self) -> None:
        header = dict(self.entries)
        if self.metadata:
            header["__metadata__"] = self.metadata
        blob = json.dumps(header, separators=(",", ":")).encode()
        if len(blob) > self.reserve:
            self.f.close()
            raise ValueError(f"{self.path}: header needs {len(blob)} bytes, reserved {self.reserve}")
        self.f.seek(0)
        self.f.write(struct.pack("<Q", self.reserve) + blob.ljust(self.reserve, b" "))
        self.f.close()
