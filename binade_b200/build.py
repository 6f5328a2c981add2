"""Builds the two native libraries in-tree (python -m binade_b200.build).

    binade_b200/lib/libbinade_b200.so       CUDA kernels + C ABI, sm_100a only
    binade_b200/lib/libbinade_b200_host.so  host codec (Rice encoder), plain C++

nvcc cross-compiles without a GPU. A library is rebuilt when any of its sources is newer.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "lib"
INCLUDE = PKG.parent / "include"
CUDA_LIB = LIBDIR / "libbinade_b200.so"
HOST_LIB = LIBDIR / "libbinade_b200_host.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]  # fmt: skip


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: the CUDA library cannot be built")


def _stale(target: Path, sources) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in sources)


def cuda_sources():
    return sorted(CSRC.glob("*.cu"))


def build(force: bool = False, verbose: bool = False) -> None:
    LIBDIR.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    cu = cuda_sources()
    if force or _stale(CUDA_LIB, cu + headers):
        cmd = [_nvcc(), *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", str(CUDA_LIB), *map(str, cu)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError("nvcc failed")
    host = [CSRC / "host_codec.cpp"]
    if force or _stale(HOST_LIB, host + headers):
        cmd = ["g++", "-O3", "-std=c++17", "-fPIC", "-shared", "-pthread", "-o", str(HOST_LIB), *map(str, host)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("g++ failed")


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(CUDA_LIB, HOST_LIB)
