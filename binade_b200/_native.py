"""ctypes loader of the two native libraries (see include/binade_b200.h).

Nothing here computes: a missing library or a non-zero status raises, there is no fallback.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

LIBDIR = Path(__file__).resolve().parent / "lib"
STATUS = {1: "bad argument", 2: "CUDA error", 3: "buffer too small", 4: "malformed stream"}
ERR_CAPACITY = 3

_vp, _i64, _u64, _int = C.c_void_p, C.c_int64, C.c_uint64, C.c_int


class R4Struct(C.Structure):
    """bn_r4: device pointers of one R4 matrix."""

    _fields_ = [(n, _vp) for n in ("raw", "codes", "flags", "esc", "table", "row_esc")] + [("n_esc", _u64), ("esc_cols", _vp), ("col_esc", _vp)]


_SIGNATURES = {
    "cuda": {
        "bn_abi_version": [],
        "bn_device_status": [C.POINTER(_int)],
        "bn_device_status_reset": [],
        "bn_set_wait_limit_ns": [_u64],
        "bn_rice_ranks": [_vp, _vp, _u64, _vp, _i64, _i64, _vp, _vp, _vp],
        "bn_rice_unpack": [_vp, _vp, _u64, _vp, _vp, _vp, _i64, _i64, _vp, _vp, _vp],
        "bn_rice_to_r4": [_vp, _vp, _u64, _vp, _vp, _i64, _i64, _vp, _vp, _vp, _vp, _u64, _vp, _vp, _vp],
        "bn_r4_finish": [_vp, _vp, _vp, _i64, _vp, _vp, _u64, _vp],
        "bn_rice_to_r4_static": [_vp, _vp, _u64, _vp, _vp, _i64, _i64, _vp, _vp, _vp, _vp, _u64, _vp, _vp],
        "bn_r4_decode": [C.POINTER(R4Struct), _i64, _i64, _i64, _i64, _i64, _vp, _vp],
        "bn_r4_esc_columns": [C.POINTER(R4Struct), _i64, _i64, _vp, _vp, _vp],
        "bn_bf16_split_hist": [_vp, _i64, _vp, _vp, _vp],
        "bn_rice_encode_plan": [_vp, _vp, _i64, _i64, _vp, _vp, _vp, _vp, _vp],
        "bn_rice_encode_write": [_vp, _vp, _vp, _vp, _i64, _i64, _vp, _u64, _vp],
        "bn_r4_lookup": [C.POINTER(R4Struct), _i64, _vp, _i64, _i64, _vp, _vp],
        "bn_rice_lookup": [_vp, _vp, _u64, _vp, _vp, _vp, _i64, _i64, _vp, _i64, _vp, _vp],
        "bn_f1_offsets": [_vp, _vp, _u64, _i64, _i64, _vp, _vp, _vp, _vp, _vp],
        "bn_f1_ranks": [_vp, _vp, _u64, _vp, _vp, _u64, _vp, _vp, _i64, _i64, _vp, _vp],
        "bn_f1_unpack": [_vp, _vp, _u64, _vp, _vp, _u64, _vp, _vp, _vp, _i64, _i64, _vp, _vp],
        "bn_f1_to_r4": [_vp, _vp, _u64, _vp, _vp, _u64, _vp, _vp, _i64, _i64, _vp, _vp, _vp, _vp, _u64, _vp, _vp, _vp],
        "bn_r4_gather_grouped": [_vp, C.POINTER(R4Struct), _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _vp, _vp, _vp],
        "bn_push_gather": [_vp, _vp, _int, _vp, _u64, _vp, _int, _int, _vp, _vp],
        "bn_push_gather_beside": [_vp, _vp, _int, _vp, _u64, _vp, _int, _int, _vp, _vp],
        "bn_r4_mma": [_vp, _i64, C.POINTER(R4Struct), _i64, _i64, _i64, _vp, _i64, _vp],
        "bn_r4_mma_split": [_vp, _i64, C.POINTER(R4Struct), _i64, _i64, _i64, _vp, _i64, _int, _vp],
        "bn_r4_rows": [_vp, _i64, C.POINTER(R4Struct), _i64, _i64, _i64, _vp, _i64, _vp],
        "bn_r4_rows_multi": [_vp, _vp, _vp, _int, _i64, _vp, _vp],
        "bn_r4_gather": [_vp, C.POINTER(R4Struct), _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _vp, _vp, _vp],
    },
    "host": {
        "bn_host_split_hist": [_vp, _i64, _vp, _vp],
        "bn_host_rank_table": [_vp, _vp, _vp],
        "bn_host_rice_encode": [_vp, _vp, _i64, _i64, _vp, _vp, _vp, _u64, C.POINTER(_u64), _int],
        "bn_host_rice_encode_ranks": [_vp, _i64, _i64, _vp, _vp, _vp, _u64, C.POINTER(_u64), _int],
        "bn_host_f1_encode": [_vp, _vp, _i64, _i64, _vp, _vp, _u64, _vp, _u64, _vp, _int],
    },
}
_FILES = {"cuda": "libbinade_b200.so", "host": "libbinade_b200_host.so"}
_ERRFN = {"cuda": "bn_last_error", "host": "bn_host_last_error"}
_libs: dict = {}


class NativeError(RuntimeError):
    def __init__(self, fn: str, status: int, detail: str):
        super().__init__(f"{fn} failed: {STATUS.get(status, status)}: {detail}")
        self.status = status


def load(which: str) -> C.CDLL:
    """The `cuda` or `host` library with argument types set; raises if it was not built."""
    if which not in _libs:
        path = LIBDIR / _FILES[which]
        if not path.exists():
            raise RuntimeError(f"{path} is missing: build it with `python -m binade_b200.build` (no CPU fallback exists)")
        lib = C.CDLL(str(path))
        for name, args in _SIGNATURES[which].items():
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = args, _int
        getattr(lib, _ERRFN[which]).restype = C.c_char_p
        _libs[which] = lib
    return _libs[which]


def call(which: str, fn: str, *args, ok=()) -> int:
    """Call an entry point; raise NativeError on a status not listed in `ok`."""
    lib = load(which)
    status = getattr(lib, fn)(*args)
    if status and status not in ok:
        raise NativeError(fn, status, getattr(lib, _ERRFN[which])().decode())
    return status


def symbols(which: str):
    return list(_SIGNATURES[which]) + [_ERRFN[which]]


def nptr(a):
    """Pointer to a contiguous numpy array (or None)."""
    return None if a is None else C.c_void_p(a.ctypes.data)
