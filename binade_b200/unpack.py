"""Reconstruct BF16 weights from a Binade model (format 2), decoding on the GPU.

    python -m binade_b200.cli unpack <packed-dir> --out DIR

Rows are decoded in chunks so memory stays bounded: each chunk's Rice stream, raw bytes and
table go to the device, one kernel rebuilds the BF16 words (decode + table lookup + join), and
every row's end is checked against the next row's offset. Same interface as the reference's
binade/unpack.py; its numpy decoder (`gpu=False`) is not part of this package.

`unpack(p)` is the tensor-level inverse of `pack.pack`.
"""

from __future__ import annotations

import argparse
import json
import math
import shutil
from pathlib import Path

import numpy as np

from . import st
from .format import TILE
from .pack import CHUNK, KNOWN_SUFFIXES


def _decode_rows(table, meta, words, roff, raw, K: int, name: str, nxt: np.ndarray) -> np.ndarray:
    """uint16 [rows, K] of one chunk; meta/roff/raw/nxt cover the chunk, words the whole tensor."""
    import torch

    from .cuda import kernels as ck

    R = roff.size
    out, rend = ck.rice_unpack(ck.to_device(meta), words, ck.to_device(roff), table, ck.to_device(raw), R, K)
    rend = rend.cpu().numpy().view(np.uint32)
    if np.any(rend.astype(np.int64) != nxt):
        raise ValueError(f"{name}: rows do not end where the next row starts")
    return out.view(torch.int16).cpu().numpy().view(np.uint16)


def unpack(p: dict) -> np.ndarray:
    """{"raw", "table", "meta", "bits", "roff"[, "shape"]} -> BF16 words with the original shape."""
    from .cuda import kernels as ck

    raw = np.ascontiguousarray(p["raw"], np.uint8)
    shape = tuple(p.get("shape", raw.shape))
    K = shape[-1]
    R = raw.size // K if K else 0
    if p["meta"].size != R * math.ceil(K / TILE) or p["roff"].size != R:
        raise ValueError(f"{p['meta'].size} tiles and {p['roff'].size} row offsets for {R} x {K}")
    if R == 0:
        return np.zeros(shape, np.uint16)
    nxt = np.append(p["roff"][1:].astype(np.int64), p["bits"].size)
    u = _decode_rows(ck.to_device(p["table"]), p["meta"], ck.to_device(p["bits"]), p["roff"], raw.reshape(R, K), K, "tensor", nxt)
    return u.reshape(shape)


class PackedModel:
    def __init__(self, path, gpu: bool = True):
        if not gpu:
            raise NotImplementedError("binade_b200 decodes on the GPU only; the CPU decoder is test infrastructure")
        self.path = Path(path)
        self.gpu = True
        self.infos = {t.name: t for t in st.list_tensors(self.path)}
        self.packed = sorted(n[:-4] for n in self.infos if n.endswith(".raw") and (f"{n[:-4]}.idx" in self.infos or f"{n[:-4]}.bits" in self.infos))

    def names(self) -> list:
        """Original tensor names, in file order."""
        parts = {f"{p}.{s}" for p in self.packed for s in KNOWN_SUFFIXES}
        stems = set(self.packed)
        out = []
        for n in self.infos:
            if n.endswith(".raw") and n[:-4] in stems:
                out.append(n[:-4])
            elif n not in parts:
                out.append(n)
        return out

    def info(self, name: str) -> st.TensorInfo:
        return self.infos[f"{name}.raw"] if name in self.packed else self.infos[name]

    def rows(self, name: str, chunk: int = CHUNK):
        """Yield (r0, r1, uint16 [r1 - r0, K]) over a packed tensor's 2-D view."""
        import torch

        from .cuda import kernels as ck

        raw = self.infos[f"{name}.raw"]
        if f"{name}.bits" not in self.infos:  # format 1: fixed-width codes, one escape stream per tensor
            table, meta, idx, esc = (st.read(self.infos[f"{name}.{s}"]) for s in ("table", "meta", "idx", "esc"))
            R, K = raw.rows, raw.shape[-1]
            f1 = ck.Format1(meta, idx, esc, table, R, K)  # offsets of every row, on the device
            step = max(1, chunk // K)
            for r0 in range(0, R, step):
                r1 = min(R, r0 + step)
                part = ck.Format1.rows_of(f1, r0, r1)
                yield r0, r1, part.unpack(st.read(raw, (r0, r1))).view(torch.int16).cpu().numpy().view(np.uint16)
            return
        table, meta, words, roff = (st.read(self.infos[f"{name}.{s}"]) for s in ("table", "meta", "bits", "roff"))
        R, K = raw.rows, raw.shape[-1]
        per_row = math.ceil(K / TILE)
        if meta.size != R * per_row or roff.size != R:
            raise ValueError(f"{name}: {meta.size} tiles and {roff.size} row offsets for {R} x {K}")
        nxt = np.append(roff[1:].astype(np.int64), words.size)
        d_table, d_words = ck.to_device(table), ck.to_device(words)
        step = max(1, chunk // K)
        for r0 in range(0, R, step):
            r1 = min(R, r0 + step)
            yield r0, r1, _decode_rows(d_table, meta[r0 * per_row : r1 * per_row], d_words, roff[r0:r1], st.read(raw, (r0, r1)), K, name, nxt[r0:r1])

    def tensor(self, name: str) -> np.ndarray:
        """Whole tensor: uint16 BF16 words for packed weights, the stored dtype otherwise."""
        if name not in self.packed:
            return st.read(self.infos[name])
        return np.concatenate([u for _, _, u in self.rows(name)]).reshape(self.info(name).shape)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("packed", help="packed model directory, or a Binade repo id on the Hugging Face Hub")
    ap.add_argument("--out", type=Path, required=True)
    args = ap.parse_args()
    packed = st.fetch(args.packed)
    pm = PackedModel(packed)
    args.out.mkdir(parents=True, exist_ok=True)
    by_file: dict = {}
    for n in pm.names():
        by_file.setdefault(pm.info(n).file.name, []).append(n)
    for fname, names in by_file.items():
        w = st.Writer(args.out / fname, sum(len(n) + 160 for n in names) + 4096)
        for n in names:
            info = pm.info(n)
            if n in pm.packed:
                w.begin(n, "BF16", info.shape)
                for _, _, u in pm.rows(n):
                    w.write(u)
                w.end()
            else:
                w.add(n, st.read(info), info.dtype)
        w.close()
    config = packed / "config.json"
    if config.exists():
        c = json.loads(config.read_text())
        c.pop("quantization_config", None)
        (args.out / "config.json").write_text(json.dumps(c, indent=2) + "\n")
    skip = {"config.json", "binade_pack.json", st.INDEX}
    for f in packed.iterdir():
        if f.is_file() and f.suffix != ".safetensors" and f.name not in skip:
            shutil.copy(f, args.out / f.name)


if __name__ == "__main__":
    main()
