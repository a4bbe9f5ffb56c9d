"""The finished pair table in a POSIX shared-memory segment (layout and C reader: ``include/ks_pairtab_shm.h``).

The reference's daemon keeps its table in string-keyed hash maps filled from ``pair_eff.tsv`` / ``kernel_us.tsv``
(scheduler/scheduler_daemon.cpp:230-274); this is the same content as sorted arrays a scheduler can map and search
without parsing: both tables (SHAPE rows and TYPE rows, as in the files), the kernel names and the models.

``publish`` writes an image with ``ks_pairtab_publish`` (host code in libks_b200.so; tmp + rename, so a visible segment
never changes); ``attach`` maps a segment and offers the daemon's two lookups (``lookup_eff``, ``kernel_us``) over numpy
views -- the Python twin of the header's inline functions.
"""
from __future__ import annotations

import ctypes
import mmap
import os

import numpy as np

from . import _lib
from .records import KEY_ROW_DTYPE, PAIR_ROW_DTYPE

SHM_NAME = "/kernel_sched_pairtab_v1"
MAGIC = 0x3154524941505348
KEY_DTYPE = np.dtype([("key", "<u8"), ("name_id", "<u4"), ("tenant", "<u4"), ("grid", "<u4", (3,)), ("block", "<u4", (3,)), ("solo_us", "<f8"), ("launches", "<u8")])
VAL_DTYPE = np.dtype([("efficiency", "<f4"), ("gangs", "<u4")])
_TABLE_DTYPE = np.dtype([("n_keys", "<u8"), ("n_rows", "<u8"), ("keys_off", "<u8"), ("row_ptr_off", "<u8"), ("cols_off", "<u8"), ("vals_off", "<u8")])
HEADER_DTYPE = np.dtype([("magic", "<u8"), ("version", "<u4"), ("reserved", "<u4"), ("total_bytes", "<u8"), ("generation", "<u8"), ("n_names", "<u8"),
                         ("names_off", "<u8"), ("n_models", "<u8"), ("models_off", "<u8"), ("shape", _TABLE_DTYPE), ("type", _TABLE_DTYPE)])


def kernel_key(name_id: int, grid, block, tenant: int, type_key: bool = False, smem: int = 0) -> int:
    """The 64-bit kernel key of a launch shape, computed on the host exactly as the device does."""
    g = (ctypes.c_uint32 * 3)(*[int(v) for v in grid])
    b = (ctypes.c_uint32 * 3)(*[int(v) for v in block])
    return int(_lib.load().ks_kernel_key(int(name_id), g, b, int(smem), int(tenant), _lib.KEY_TYPE if type_key else 0))


def publish(shape_tables, type_tables, names, models, name: str = SHM_NAME, generation: int = 1) -> int:
    """shape_tables / type_tables: (key_rows, pair_rows) structured arrays of the two tables; names[name_id], models[tenant].
    Returns the size of the image in bytes."""
    lib = _lib.load()
    arrays = []
    for keys, pairs in (shape_tables, type_tables):
        arrays += [np.ascontiguousarray(keys, dtype=KEY_ROW_DTYPE), np.ascontiguousarray(pairs, dtype=PAIR_ROW_DTYPE)]
    c_names = (ctypes.c_char_p * max(len(names), 1))(*[str(s).encode() for s in names])
    c_models = (ctypes.c_char_p * max(len(models), 1))(*[str(s).encode() for s in models])
    r = lib.ks_pairtab_publish(name.encode(), _lib.ptr(arrays[0]), len(arrays[0]), _lib.ptr(arrays[1]), len(arrays[1]), _lib.ptr(arrays[2]), len(arrays[2]),
                               _lib.ptr(arrays[3]), len(arrays[3]), c_names, len(names), c_models, len(models), int(generation))
    if r < 0:
        raise _lib.KsError(int(-r), lib.ks_pairtab_last_error().decode())
    return int(r)


def unlink(name: str = SHM_NAME) -> None:
    _lib.load().ks_pairtab_unlink(name.encode())


class _Table:
    def __init__(self, buf, desc):
        n_keys, n_rows = int(desc["n_keys"]), int(desc["n_rows"])
        self.keys = np.frombuffer(buf, dtype=KEY_DTYPE, count=n_keys, offset=int(desc["keys_off"]))
        self.row_ptr = np.frombuffer(buf, dtype="<u4", count=n_keys + 1, offset=int(desc["row_ptr_off"]))
        self.cols = np.frombuffer(buf, dtype="<u4", count=n_rows, offset=int(desc["cols_off"]))
        self.vals = np.frombuffer(buf, dtype=VAL_DTYPE, count=n_rows, offset=int(desc["vals_off"]))

    def find_key(self, key: int) -> int:
        i = int(np.searchsorted(self.keys["key"], np.uint64(key)))
        return i if i < len(self.keys) and int(self.keys["key"][i]) == int(key) else -1

    def find_pair(self, key_x: int, key_y: int):
        ix, iy = self.find_key(key_x), self.find_key(key_y)
        if ix < 0 or iy < 0:
            return None
        if self.keys["tenant"][ix] > self.keys["tenant"][iy]:
            ix, iy = iy, ix
        lo, hi = int(self.row_ptr[ix]), int(self.row_ptr[ix + 1])
        j = lo + int(np.searchsorted(self.cols[lo:hi], iy))
        if j >= hi or int(self.cols[j]) != iy:
            return None
        return np.float32(self.vals["efficiency"][j]), int(self.vals["gangs"][j])  # copies: nothing keeps the mapping alive


class Attached:
    """A mapped segment.  ``close()`` (or the context manager) unmaps it."""

    def __init__(self, name: str = SHM_NAME):
        fd = os.open("/dev/shm" + name, os.O_RDONLY)
        try:
            self._map = mmap.mmap(fd, 0, prot=mmap.PROT_READ)
        finally:
            os.close(fd)
        hd = np.frombuffer(self._map, dtype=HEADER_DTYPE, count=1)[0]
        if int(hd["magic"]) != MAGIC or int(hd["version"]) != 1 or int(hd["total_bytes"]) > len(self._map):
            raise ValueError(f"{name} is not a version-1 pair table segment")
        self.generation = int(hd["generation"])
        self.names = self._strings(int(hd["names_off"]), int(hd["n_names"]))
        self.models = self._strings(int(hd["models_off"]), int(hd["n_models"]))
        self.shape = _Table(self._map, hd["shape"])
        self.type = _Table(self._map, hd["type"])

    def _strings(self, off, n):
        offs = np.frombuffer(self._map, dtype="<u8", count=n + 1, offset=off)
        return [bytes(self._map[int(offs[i]): int(offs[i + 1])]).decode() for i in range(n)]

    def lookup_eff(self, shape_a: int, shape_b: int, type_a: int, type_b: int, min_gangs: int = 1):
        """scheduler_daemon.cpp:269-274: the shape-pair row if at least ``min_gangs`` gangs measured it, else the type-pair
        row; -> (efficiency, gangs) or None."""
        s = self.shape.find_pair(shape_a, shape_b)
        if s is not None and s[1] >= min_gangs:
            return s
        return self.type.find_pair(type_a, type_b)

    def kernel_us(self, shape_key: int, type_key: int) -> float:
        i = self.shape.find_key(shape_key)
        if i >= 0 and not np.isnan(self.shape.keys["solo_us"][i]):
            return float(self.shape.keys["solo_us"][i])
        i = self.type.find_key(type_key)
        return float(self.type.keys["solo_us"][i]) if i >= 0 else float("nan")

    def close(self):
        self.shape = self.type = None
        try:
            self._map.close()
        except BufferError:  # a caller still holds a view of the arrays: the mapping goes when the view does
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
