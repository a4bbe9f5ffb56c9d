"""ctypes binding of libks_b200.so.

Follows the reference's own binding convention (scheduler/sched_hooks.py:36-59): one table of
(name, argument types, return type) that must match the library's ``extern "C"`` functions, and a loader that
refuses a library lacking any of them.  There is no fallback: if the library is missing or a call fails the
caller gets an exception, never a CPU result.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_double, c_int, c_int64, c_uint32, c_uint64, c_void_p
from pathlib import Path

import numpy as np

LIB_PATH = Path(__file__).resolve().parent / "libks_b200.so"

# flags (include/ks_b200.h)
ON_DEVICE = 1
ASSUME_TIME_ORDERED = 2
KEY_TYPE = 4
TIMING = 8

ERR_ARG, ERR_CUDA, ERR_RECORD, ERR_NOT_ORDERED, ERR_TOO_MANY_KEYS = 1, 2, 3, 4, 5
ERR_TABLE_FULL, ERR_CAPACITY, ERR_WAIT, ERR_DUPLICATE, ERR_TOO_LARGE, ERR_COMM = 6, 7, 8, 9, 10, 11
ERR_REBUILD = 12
COL_U64, COL_MILLI, COL_DIMS, COL_HASH, COL_SPAN = 0, 1, 2, 3, 4


class KsConfig(ctypes.Structure):
    _fields_ = [("max_records", c_uint64), ("max_pairs", c_uint64), ("max_pair_rows", c_uint32), ("reserved", c_uint32)]


class KsSynthTenant(ctypes.Structure):
    _fields_ = [("n_keys", c_uint32), ("tenant", c_uint32), ("name_id", c_void_p), ("grid", c_void_p), ("block", c_void_p), ("smem", c_void_p),
                ("dur_ns", c_void_p), ("cdf", c_void_p), ("n_launches", c_uint64), ("gap_mean_ns", c_double)]


class KsTableInfo(ctypes.Structure):
    _fields_ = [
        ("n_records", c_uint64), ("n_keys", c_uint64), ("n_solo", c_uint64), ("n_pairs", c_uint64), ("n_rows", c_uint64),
        ("max_duration_ns", c_uint64), ("min_start_ns", c_uint64), ("max_start_ns", c_uint64),
        ("was_time_ordered", c_uint32), ("sort_passes", c_uint32),
        ("ms_stage_in", ctypes.c_float), ("ms_decode", ctypes.c_float), ("ms_order", ctypes.c_float), ("ms_dict", ctypes.c_float),
        ("ms_join", ctypes.c_float), ("ms_sort", ctypes.c_float), ("ms_reduce", ctypes.c_float), ("ms_finalize", ctypes.c_float),
        ("ms_total", ctypes.c_float), ("ms_sort_pass", ctypes.c_float),
    ]

    def as_dict(self):
        return {name: getattr(self, name) for name, _ in self._fields_ if not name.startswith("reserved")}


# Everything called in libks_b200.so: (name, argument types, return type) -- must match include/ks_b200.h.
KS_API = [
    ("ks_version", [], c_int),
    ("ks_status_string", [c_int], c_char_p),
    ("ks_create", [c_int, c_void_p, POINTER(KsConfig)], c_void_p),
    ("ks_destroy", [c_void_p], None),
    ("ks_last_error", [c_void_p], c_char_p),
    ("ks_stream", [c_void_p], c_void_p),
    ("ks_launch_count", [c_void_p], c_uint64),
    ("ks_pinned_alloc", [c_uint64], c_void_p),
    ("ks_pinned_free", [c_void_p], None),
    ("ks_build_table", [c_void_p, c_void_p, c_uint64, c_uint32, POINTER(KsTableInfo)], c_int64),
    ("ks_build_table_streamed", [c_void_p, c_void_p, c_uint64, c_uint32, c_uint64, c_uint32, POINTER(KsTableInfo)], c_int64),
    ("ks_selftest_bounded_wait", [c_void_p], c_int64),
    ("ks_copy_pair_rows", [c_void_p, c_void_p, c_uint64, c_uint32], c_int64),
    ("ks_copy_key_rows", [c_void_p, c_void_p, c_uint64, c_uint32], c_int64),
    ("ks_hash_keys", [c_void_p, c_void_p, c_uint64, c_uint32, c_void_p], c_int64),
    ("ks_sort_pairs_u64", [c_void_p, c_void_p, c_void_p, c_uint64, c_int, c_int, c_uint32], c_int64),
    ("ks_sort_pairs_u32", [c_void_p, c_void_p, c_void_p, c_uint64, c_int, c_int, c_uint32], c_int64),
    ("ks_sort_pairs_u32_noalloc", [c_void_p, c_void_p, c_void_p, c_uint64, c_int, c_int], c_int64),
    ("ks_sort_launches", [c_void_p, c_void_p, c_uint64, c_uint32, c_void_p, c_void_p], c_int64),
    ("ks_join_overlaps", [c_void_p, c_void_p, c_uint64, c_uint32, c_void_p, c_void_p, c_uint64], c_int64),
    ("ks_segment_stats", [c_void_p, c_void_p, c_void_p, c_uint64, c_uint32, c_void_p], c_int64),
    ("ks_count_batches", [c_void_p, c_void_p, c_uint64, c_void_p, c_uint64, c_uint32, POINTER(c_uint64)], c_int64),
    ("ks_combine_duplicates", [c_void_p, c_void_p, c_void_p, c_void_p, c_uint64, c_uint32, c_uint32, c_uint32, c_void_p, c_void_p], c_int64),
    ("ks_pool_launches", [c_void_p, c_void_p, c_void_p, c_uint64, c_uint32, c_uint32, c_uint32, c_void_p, c_void_p, c_void_p], c_int64),
    ("ks_mg_begin", [c_void_p, c_void_p, c_uint64, c_uint32], c_int64),
    ("ks_mg_tail", [c_void_p, c_void_p, c_uint64], c_int64),
    ("ks_mg_halo", [c_void_p, c_void_p, c_uint64], c_int64),
    ("ks_mg_local_keys", [c_void_p, c_void_p, c_void_p, c_uint64], c_int64),
    ("ks_mg_global_keys", [c_void_p, c_void_p, c_void_p, c_uint64], c_int64),
    ("ks_mg_counts", [c_void_p, c_void_p, c_void_p, c_int], c_int64),
    ("ks_mg_samples", [c_void_p], c_int64),
    ("ks_mg_key_histogram", [c_void_p, c_void_p, POINTER(c_uint32)], c_int64),
    ("ks_mg_partition", [c_void_p, POINTER(c_uint32), c_uint32, c_uint32, c_void_p, c_uint64, POINTER(c_uint64)], c_int64),
    ("ks_mg_reduce", [c_void_p, c_void_p, c_uint64], c_int64),
    ("ks_mg_row_count", [c_void_p], c_int64),
    ("ks_mg_solo", [c_void_p, c_void_p, c_int], c_int64),
    ("ks_mg_finalize", [c_void_p], c_int64),
    ("ks_mg_unique_id", [c_void_p], c_int),
    ("ks_mg_comm_init", [c_void_p, c_void_p, c_int, c_int], c_int),
    ("ks_mg_build", [c_void_p, c_void_p, c_uint64, c_uint32, POINTER(KsTableInfo)], c_int64),
    ("ks_mg_comm_destroy", [c_void_p], c_int),
    ("ks_mg_peer_memory", [c_void_p], c_int),
    ("ks_tsv_parse", [c_void_p, c_void_p, c_uint64, c_uint32], c_int64),
    ("ks_tsv_dictionary", [c_void_p, c_int, c_void_p, c_void_p], c_int64),
    ("ks_tsv_label", [c_void_p, c_void_p, c_uint64, c_uint64, c_uint32], c_int64),
    ("ks_tsv_extract", [c_void_p, c_void_p, c_uint64, c_uint32, POINTER(c_uint32), POINTER(c_uint32), c_void_p, c_uint64, c_uint32], c_int64),
    ("ks_segment_hist", [c_void_p, c_void_p, c_void_p, c_uint64, c_uint32, c_uint32, c_uint32, c_void_p], c_int64),
    ("ks_tsv_finish", [c_void_p, c_void_p, c_void_p, c_uint32, c_void_p, c_uint64, c_uint32], c_int64),
    ("ks_function_base", [c_char_p, c_char_p, c_uint64], c_int64),
    ("ks_update_begin", [c_void_p, c_uint32], c_int64),
    ("ks_update", [c_void_p, c_void_p, c_uint64, c_uint32, POINTER(KsTableInfo)], c_int64),
    ("ks_update_table", [c_void_p], c_int64),
    ("ks_update_end", [c_void_p], c_int64),
    ("ks_kernel_key", [c_uint32, POINTER(c_uint32), POINTER(c_uint32), c_uint32, c_uint32, c_uint32], c_uint64),
    ("ks_pairtab_publish", [c_char_p, c_void_p, c_uint64, c_void_p, c_uint64, c_void_p, c_uint64, c_void_p, c_uint64, POINTER(c_char_p), c_uint64,
                            POINTER(c_char_p), c_uint64, c_uint64], c_int64),
    ("ks_synth_trace", [POINTER(KsSynthTenant), c_uint32, c_double, c_double, c_double, c_uint64, c_uint64, c_void_p, c_uint64, c_uint32, c_uint32], c_int64),
    ("ks_pairtab_unlink", [c_char_p], c_int),
    ("ks_pairtab_last_error", [], c_char_p),
]

_lib = None


class KsError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"libks_b200: status {status}: {message}")
        self.status = status


def load(path=None):
    """Loads libks_b200.so and declares the signatures; raises if the library or a symbol is missing."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = Path(path or os.environ.get("KS_B200_LIB") or LIB_PATH)
    if not p.exists():
        raise RuntimeError(f"{p} is not built: run `python -m kernel_scheduling_b200.build` (there is no CPU fallback)")
    lib = ctypes.CDLL(str(p))
    missing = [name for name, _, _ in KS_API if not hasattr(lib, name)]
    if missing:
        raise RuntimeError(f"{p} does not export {', '.join(missing)}: is it built from the csrc/ that matches this package?")
    for name, argtypes, restype in KS_API:
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = restype
    if path is None:
        _lib = lib
    return lib


def ptr(a):
    """Address of a numpy array's buffer (or a raw integer device pointer)."""
    if a is None:
        return None
    if isinstance(a, int):
        return c_void_p(a)
    assert a.flags["C_CONTIGUOUS"]
    return c_void_p(a.ctypes.data)


def function_base(symbol: str) -> str:
    """Short kernel name of a (mangled) symbol: scheduler/kernel_key.hpp:13-55."""
    lib = load()
    buf = ctypes.create_string_buffer(max(4096, 4 * len(symbol) + 64))
    r = lib.ks_function_base(symbol.encode(), buf, len(buf))
    if r < 0:
        raise KsError(int(-r), "ks_function_base")
    return buf.value.decode()
