"""Packer: BF16 safetensors model -> Binade model (format 2, Rice).

    python -m binade_b200.cli pack <model-dir> --out DIR [--classes linear,embed,ple,mm]

Streams one tensor at a time. A packed weight `name` becomes name.raw (sign + mantissa bytes,
original shape), name.table (exponent by rank), name.meta (one byte per tile), name.bits (Rice
stream, uint32 words) and name.roff (first word of each row); everything else is copied byte
for byte, shard names follow the input. Output files are byte-identical to those of the
reference's packer (binade/pack.py) for format 2; the encoder itself is C++ on all host cores.

`pack(w)` is the tensor-level form: BF16 words [.., K] -> dict of the five arrays.
"""

from __future__ import annotations

import argparse
import json
import shutil
import subprocess
import time
from pathlib import Path

import numpy as np

from . import _native, rice, st
from .classify import MIN_DIM, classify
from .format import TILE, encode_words as f1_encode_words, rank_table

VERSION = "2"
CLASSES = ("linear", "embed", "ple", "mm")
CHUNK = 1 << 24  # weights per read
PARTS = {"1": ("raw", "table", "meta", "idx", "esc"), "2": ("raw", "table", "meta", "bits", "roff")}
KNOWN_SUFFIXES = ("raw", "table", "meta", "idx", "esc", "bits", "roff")  # of either on-disk format
REPO = Path(__file__).resolve().parents[1]


def quant(version: str = VERSION) -> dict:
    return {"quant_method": "binade", "version": version, "tile": TILE}


def pack_meta(path) -> dict | None:
    """The Binade marker of a packed directory: the "binade" entry of binade_pack.json, else a
    quantization_config in config.json (older packs); None if the directory is not a pack."""
    path = Path(path)
    report = path / "binade_pack.json"
    if report.exists():
        marker = json.loads(report.read_text()).get("binade")
        if marker and marker.get("quant_method") == "binade":
            return marker
    config = path / "config.json"
    if config.exists():
        q = json.loads(config.read_text()).get("quantization_config", {})
        if q.get("quant_method") == "binade":
            return q
    return None


def packable(info: st.TensorInfo, classes) -> bool:
    """BF16, 2-D or 3-D, of a requested class; vision/audio tensors only at linear-weight sizes."""
    if info.dtype != "BF16" or len(info.shape) not in (2, 3):
        return False
    k = classify(info.name, info.shape, info.dtype)
    if k.cls not in classes:
        return False
    return k.cls != "mm" or min(info.shape[-2:]) >= MIN_DIM


def spans(info: st.TensorInfo, chunk: int = CHUNK):
    """Row ranges of about `chunk` weights each."""
    step = max(1, chunk // info.shape[-1])
    return [(r, min(info.rows, r + step)) for r in range(0, info.rows, step)]


def _histogram(u: np.ndarray, hist: np.ndarray) -> None:
    _native.call("host", "bn_host_split_hist", _native.nptr(u), u.size, None, _native.nptr(hist))


def _raw(u: np.ndarray) -> np.ndarray:
    out = np.empty(u.shape, np.uint8)
    scratch = np.zeros(256, np.int64)
    _native.call("host", "bn_host_split_hist", _native.nptr(u), u.size, _native.nptr(out), _native.nptr(scratch))
    return out


def pack(w: np.ndarray, chunk: int = CHUNK, gpu: bool = False) -> dict:
    """BF16 words (uint16, [.., K]) -> {"raw", "table", "meta", "bits", "roff", "shape"}.
    gpu: encode on the CUDA device (the same arrays, bit for bit; the reference and the default
    path encode on host cores)."""
    w = np.ascontiguousarray(w, np.uint16)
    if gpu:
        from .cuda import kernels as ck

        d = ck.rice_encode(ck.to_device(w.view(np.int16)))
        host = lambda t, dt: t.cpu().numpy().view(dt)
        return {"raw": host(d["raw"], np.uint8).reshape(w.shape), "table": host(d["table"], np.uint8), "meta": host(d["meta"], np.uint8), "bits": host(d["bits"], np.uint32), "roff": host(d["roff"], np.uint32), "shape": tuple(w.shape)}
    rows = w.reshape(-1, w.shape[-1])
    hist = np.zeros(256, np.int64)
    _histogram(rows, hist)
    table, rank = rank_table(hist)
    meta, bits, roff = rice.encode_words(rows, rank)
    return {"raw": _raw(w), "table": table, "meta": meta, "bits": bits, "roff": roff, "shape": tuple(w.shape)}


def bits_per_weight(p: dict) -> float:
    """File bits per weight of one packed tensor (reference accounting, binade/pack.py:103)."""
    numel = int(np.prod(p["shape"]))
    return (8 * numel + 8 * p["table"].size + 8 * p["meta"].size + 32 * p["bits"].size + 32 * p["roff"].size) / numel


def pack_tensor(w: st.Writer, info: st.TensorInfo, chunk: int = CHUNK, version: str = VERSION, gpu: bool = False) -> dict:
    """gpu: histogram, raw bytes and the Rice streams on the CUDA device (the same bytes; format 2
    only). version "1": fixed-width codes with escapes (binade/format.py), encoded on host cores."""
    if version not in PARTS:
        raise ValueError(f"unknown Binade format {version!r}")
    if version == "1":
        return _pack_tensor_f1(w, info, chunk)
    if gpu:
        from .cuda import kernels as ck
    hist = np.zeros(256, np.int64)
    for span in spans(info, chunk):
        u = np.ascontiguousarray(st.read(info, span))
        if gpu:
            hist += ck.split_hist(ck.to_device(u.view(np.int16)))[1]
        else:
            _histogram(u, hist)
    table, rank = rank_table(hist)
    metas, streams, offsets, base = [], [], [], 0
    w.begin(info.name + ".raw", "U8", info.shape)
    for span in spans(info, chunk):
        u = np.ascontiguousarray(st.read(info, span))
        if gpu:
            d = ck.to_device(u.view(np.int16))
            w.write(ck.split_hist(d)[0].cpu().numpy().reshape(u.shape))
            meta, words, roff = (t.cpu().numpy() for t in ck.rice_encode_ranked(d, ck.to_device(rank)))
            words, roff = words.view(np.uint32), roff.view(np.uint32)
        else:
            w.write(_raw(u))
            meta, words, roff = rice.encode_words(u, rank)
        metas.append(meta)
        streams.append(words)
        offsets.append(roff.astype(np.uint64) + np.uint64(base))
        base += words.size
    w.end()
    if base >= 1 << 32:
        raise ValueError(f"{info.name}: {base} words overflow uint32 row offsets")
    meta, words, roff = np.concatenate(metas), np.concatenate(streams), np.concatenate(offsets).astype(np.uint32)
    w.add(info.name + ".table", table)
    w.add(info.name + ".meta", meta)
    w.add(info.name + ".bits", words)
    w.add(info.name + ".roff", roff)
    bits = 8 * info.numel + 8 * table.size + 8 * meta.size + 32 * words.size + 32 * roff.size
    return {"numel": info.numel, "distinct": int((hist > 0).sum()), "ntiles": int(meta.size), "bits": bits}


def _pack_tensor_f1(w: st.Writer, info: st.TensorInfo, chunk: int = CHUNK) -> dict:
    """Format 1 of one tensor: raw, table, meta, idx, esc (reference: binade/pack.py:72-93). Tiles
    are whole per row, so the spans' arrays simply follow each other."""
    hist = np.zeros(256, np.int64)
    for span in spans(info, chunk):
        _histogram(np.ascontiguousarray(st.read(info, span)), hist)
    table, rank = rank_table(hist)
    metas, words, escapes = [], [], []
    w.begin(info.name + ".raw", "U8", info.shape)
    for span in spans(info, chunk):
        u = np.ascontiguousarray(st.read(info, span))
        w.write(_raw(u))
        meta, idx, esc = f1_encode_words(u, rank)
        metas.append(meta), words.append(idx), escapes.append(esc)
    w.end()
    meta, idx, esc = np.concatenate(metas), np.concatenate(words), np.concatenate(escapes)
    w.add(info.name + ".table", table)
    w.add(info.name + ".meta", meta)
    w.add(info.name + ".idx", idx)
    w.add(info.name + ".esc", esc)
    bits = 8 * info.numel + 8 * table.size + 8 * meta.size + 32 * idx.size + 8 * esc.size
    return {"numel": info.numel, "distinct": int((hist > 0).sum()), "ntiles": int(meta.size), "escapes": int(esc.size), "bits": bits}


def copy_tensor(w: st.Writer, info: st.TensorInfo, chunk: int = CHUNK) -> None:
    w.begin(info.name, info.dtype, info.shape)
    if len(info.shape) < 2:
        w.write(st.read(info))
    else:
        for span in spans(info, chunk):
            w.write(st.read(info, span))
    w.end()


def _header_room(infos, classes, metadata, version) -> int:
    """Bytes to keep free for the header: a generous allowance per output tensor."""
    per = len(PARTS[version])
    room = sum((len(i.name) + 160) * (per if packable(i, classes) else 1) for i in infos)
    return room + len(json.dumps(metadata)) + 4096


def pack_model(src: Path, out: Path, classes=CLASSES, chunk: int = CHUNK, log=print, version: str = VERSION, gpu: bool = False) -> dict:
    if version not in PARTS:
        raise ValueError(f"unknown Binade format {version!r}")
    if version == "1" and gpu:
        raise ValueError("the GPU encoder writes format 2 only")
    src, out = Path(src), Path(out)
    started = time.perf_counter()
    out.mkdir(parents=True, exist_ok=True)
    infos = st.list_tensors(src)
    need, free = sum(i.nbytes for i in infos), shutil.disk_usage(out).free
    if free < need:
        raise OSError(f"{out}: {free / 1e9:.1f} GB free, packing may need up to {need / 1e9:.1f} GB")
    weight_map, stats = {}, {}
    for shard in st.shard_files(src):
        mine = [i for i in infos if i.file == shard]
        packed = {i.name: list(i.shape) for i in mine if packable(i, classes)}
        metadata = {"format": "binade", "binade_version": version, "binade_tile": str(TILE), "binade_tensors": json.dumps(packed)}
        writer = st.Writer(out / shard.name, _header_room(mine, classes, metadata, version), metadata)
        for info in mine:
            t0 = time.perf_counter()
            if info.name in packed:
                stats[info.name] = pack_tensor(writer, info, chunk, version, gpu)
                written = [f"{info.name}.{s}" for s in PARTS[version]]
                log(f"packed {info.name} {info.shape}: {stats[info.name]['bits'] / info.numel:.3f} bits/weight, {time.perf_counter() - t0:.1f}s")
            else:
                copy_tensor(writer, info, chunk)
                written = [info.name]
            for n in written:
                weight_map[n] = shard.name
        writer.close()
    # config.json stays the original model's: the marker lives in binade_pack.json
    for f in src.iterdir():
        if f.is_file() and f.suffix != ".safetensors" and f.name != st.INDEX:
            shutil.copy(f, out / f.name)
    total = sum((out / f).stat().st_size for f in sorted(set(weight_map.values())))
    (out / st.INDEX).write_text(json.dumps({"metadata": {"total_size": total}, "weight_map": weight_map}, indent=1) + "\n")
    commit = subprocess.run(["git", "rev-parse", "HEAD"], cwd=REPO, capture_output=True, text=True).stdout.strip()
    report = {
        "source": st.provenance(src),
        "binade": quant(version),
        "classes": list(classes),
        "git": commit,
        "seconds": time.perf_counter() - started,
        "input_bytes": sum(f.stat().st_size for f in st.shard_files(src)),
        "output_bytes": total,
        "packed_numel": sum(t["numel"] for t in stats.values()),
        "packed_bits": sum(t["bits"] for t in stats.values()),
        "tensors": stats,
    }
    (out / "binade_pack.json").write_text(json.dumps(report, indent=1) + "\n")
    return report


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("model")
    ap.add_argument("--out", type=Path, required=True)
    ap.add_argument("--revision")
    ap.add_argument("--classes", default=",".join(CLASSES))
    ap.add_argument("--format", default=VERSION, choices=sorted(PARTS), help="2: Rice (smaller; decoded to R4 at load), 1: fixed-width codes with escapes")
    ap.add_argument("--gpu", action="store_true", help="encode on the CUDA device instead of the host cores (same bytes)")
    args = ap.parse_args()
    r = pack_model(st.resolve(args.model, args.revision), args.out, tuple(args.classes.split(",")), version=args.format, gpu=args.gpu)
    print(
        f"{r['input_bytes'] / 1e9:.2f} GB -> {r['output_bytes'] / 1e9:.2f} GB ({r['output_bytes'] / r['input_bytes']:.1%}); "
        f"packed weights {r['packed_bits'] / r['packed_numel']:.3f} bits/weight; {r['seconds'] / 60:.1f} min"
    )


if __name__ == "__main__":
    main()
