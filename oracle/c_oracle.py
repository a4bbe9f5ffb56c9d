"""ctypes face of oracle/pair_table_oracle.c.  TEST INFRASTRUCTURE, NOT A PRODUCT PATH.

``build_pair_table`` returns the same two dicts of numpy columns as ``oracle.pair_table_oracle.build_pair_table``
(the numpy oracle it is kept equal to), fast enough for traces of 10^8 launches.  ``build()`` compiles the C file with
gcc next to this module (libks_oracle.so, git-ignored); a prebuilt library newer than the source is used as it is.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
SRC = HERE / "pair_table_oracle.c"
LIB = HERE / "libks_oracle.so"
KEY_SHAPE, KEY_TYPE = 0, 1

_U64P, _U32P, _F64P = C.POINTER(C.c_uint64), C.POINTER(C.c_uint32), C.POINTER(C.c_double)
_KEY_COLS = (("key", _U64P, 1), ("name_id", _U32P, 1), ("grid", _U32P, 3), ("block", _U32P, 3), ("smem", _U32P, 1), ("tenant", _U32P, 1),
             ("launches", _U64P, 1), ("solo_launches", _U64P, 1), ("solo_ns", _F64P, 1))
_PAIR_COLS = (("key_a", _U64P), ("key_b", _U64P), ("count", _U64P), ("flags", _U64P), ("span_sum_ns", _U64P),
              ("sum_a", _F64P), ("mean_a", _F64P), ("min_a", _F64P), ("max_a", _F64P), ("median_a", _F64P),
              ("sum_b", _F64P), ("mean_b", _F64P), ("min_b", _F64P), ("max_b", _F64P), ("median_b", _F64P), ("efficiency", _F64P))


class _Table(C.Structure):
    _fields_ = ([("n_keys", C.c_uint64), ("n_rows", C.c_uint64), ("n_pairs", C.c_uint64)]
                + [(name, typ) for name, typ, _ in _KEY_COLS] + [(name, typ) for name, typ in _PAIR_COLS])


def build(force: bool = False) -> Path:
    if not force and LIB.exists() and LIB.stat().st_mtime >= SRC.stat().st_mtime:
        return LIB
    subprocess.run(["gcc", "-O2", "-fopenmp", "-shared", "-fPIC", "-o", str(LIB), str(SRC), "-lm"], check=True)
    return LIB


_lib = None


def _load():
    global _lib
    if _lib is None:
        _lib = C.CDLL(str(build()))
        _lib.kso_build_pair_table.argtypes = [C.c_void_p, C.c_uint64, C.c_int, C.c_int, C.POINTER(_Table)]
        _lib.kso_build_pair_table.restype = C.c_int
        _lib.kso_free.argtypes = [C.POINTER(_Table)]
        _lib.kso_free.restype = None
        _lib.kso_kernel_keys.argtypes = [C.c_void_p, C.c_uint64, C.c_int, C.c_void_p]
        _lib.kso_kernel_keys.restype = None
    return _lib


def _column(ptr, count, width=1):
    if count == 0:
        return np.zeros((0, width) if width > 1 else 0, dtype=np.ctypeslib.as_array(ptr, shape=(1,)).dtype)
    a = np.ctypeslib.as_array(ptr, shape=(count * width,)).copy()
    return a.reshape(count, width) if width > 1 else a


def kernel_keys(records: np.ndarray, key_mode: int = KEY_SHAPE) -> np.ndarray:
    rec = np.ascontiguousarray(records)
    out = np.empty(len(rec), dtype=np.uint64)
    _load().kso_kernel_keys(rec.ctypes.data, len(rec), int(key_mode), out.ctypes.data)
    return out


def build_pair_table(records: np.ndarray, key_mode: int = KEY_SHAPE, threads: int = 0):
    """records (48-byte launch records, any order) -> (key_rows, pair_rows), dicts of numpy columns.

    ``threads`` = 0 uses every host core OpenMP offers.  Raises ValueError for a bad record, as the numpy oracle does.
    """
    rec = np.ascontiguousarray(records)
    assert rec.dtype.itemsize == 48
    t = _Table()
    st = _load().kso_build_pair_table(rec.ctypes.data, len(rec), int(key_mode), int(threads), C.byref(t))
    if st == -1:
        raise ValueError("record with end_ns < start_ns")
    if st == -2:
        raise ValueError("record with a duration of 2**31 ns or more")
    if st:
        raise RuntimeError(f"kso_build_pair_table failed with status {st}")
    try:
        keys = {name: _column(getattr(t, name), t.n_keys, width) for name, _, width in _KEY_COLS}
        pairs = {name: _column(getattr(t, name), t.n_rows) for name, _ in _PAIR_COLS}
    finally:
        _lib.kso_free(C.byref(t))
    return keys, pairs


def host_threads() -> int:
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
