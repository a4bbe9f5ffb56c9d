"""Host-side face of the trace -> interference-table path.

``PairTableBuilder`` wraps one library handle (one CUDA stream).  ``build`` takes the launch records (a numpy
array of RECORD_DTYPE in host memory, or a device pointer) and returns the two tables the reference's daemon
consumes (scheduler/scheduler_daemon.cpp:193-202): one row per kernel key with its solo time, one row per
pair of keys with count, slowdown statistics of both sides and the efficiency.  ``write_tsv`` emits them as
``kernel_us.tsv`` / ``pair_eff.tsv`` in the layout ``load_kernel_us`` / ``load_pair_eff`` read (:230-264).
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import _lib
from .records import KEY_ROW_DTYPE, PAIR_ROW_DTYPE, RECORD_DTYPE


class PairTableBuilder:
    def __init__(self, device: int = 0, stream: int | None = None, max_records: int = 0, max_pairs: int = 0, max_pair_rows: int = 0):
        self._lib = _lib.load()
        cfg = _lib.KsConfig(max_records, max_pairs, max_pair_rows, 0)
        self._h = self._lib.ks_create(device, ctypes.c_void_p(stream) if stream else None, ctypes.byref(cfg))
        if not self._h:
            raise _lib.KsError(_lib.ERR_CUDA, self._lib.ks_last_error(None).decode() or "ks_create failed (no CUDA device?)")
        self.info = None
        self._pinned_bufs = {}

    # -- plumbing
    def close(self):
        if getattr(self, "_h", None):
            for p, _ in self._pinned_bufs.values():
                self._lib.ks_pinned_free(p)
            self._pinned_bufs = {}
            self._lib.ks_destroy(self._h)
            self._h = None

    __del__ = close

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    @property
    def stream(self) -> int:
        return int(self._lib.ks_stream(self._h) or 0)

    @property
    def launch_count(self) -> int:
        return int(self._lib.ks_launch_count(self._h))

    def _check(self, r, what):
        if r < 0:
            raise _lib.KsError(int(-r), f"{what}: {self._lib.ks_last_error(self._h).decode()}")
        return int(r)

    @staticmethod
    def _records_arg(records, n):
        if isinstance(records, int):
            if n is None:
                raise ValueError("n is required with a device pointer")
            return ctypes.c_void_p(records), int(n), _lib.ON_DEVICE
        rec = np.ascontiguousarray(records, dtype=RECORD_DTYPE)
        return _lib.ptr(rec), len(rec), 0, rec

    # -- the whole path
    def build_device(self, records, n=None, time_ordered: bool = False, key_type: bool = False) -> int:
        """Runs the pipeline and leaves the tables on the device; returns the number of pair rows."""
        arg = self._records_arg(records, n)
        flags = arg[2] | (_lib.ASSUME_TIME_ORDERED if time_ordered else 0) | (_lib.KEY_TYPE if key_type else 0)
        info = _lib.KsTableInfo()
        rows = self._check(self._lib.ks_build_table(self._h, arg[0], arg[1], flags, ctypes.byref(info)), "ks_build_table")
        self.info = info.as_dict()
        return rows

    def build_streamed_device(self, records, n=None, window_records: int = 0, n_parts: int = 0, key_type: bool = False) -> int:
        """The same table for traces whose overlapping pairs do not fit one call: joined window after window, the samples
        kept in ``n_parts`` key ranges that are sorted and reduced one after the other (``ks_build_table_streamed``).
        Records in start order.  Returns the number of pair rows; ``fetch`` copies the tables out."""
        arg = self._records_arg(records, n)
        flags = arg[2] | (_lib.KEY_TYPE if key_type else 0)
        info = _lib.KsTableInfo()
        rows = self._check(self._lib.ks_build_table_streamed(self._h, arg[0], arg[1], flags, int(window_records), int(n_parts), ctypes.byref(info)),
                           "ks_build_table_streamed")
        self.info = info.as_dict()
        return rows

    def _pinned(self, slot: str, n: int, dtype) -> np.ndarray:
        """A page-locked array owned by the builder (grown on demand, reused by later calls)."""
        need = max(n, 1) * dtype.itemsize
        cur = self._pinned_bufs.get(slot)
        if cur is None or cur[1] < need:
            if cur is not None:
                self._lib.ks_pinned_free(cur[0])
            size = need + need // 4
            p = self._lib.ks_pinned_alloc(size)
            if not p:
                raise _lib.KsError(_lib.ERR_CUDA, "ks_pinned_alloc failed")
            cur = self._pinned_bufs[slot] = (p, size)
        raw = (ctypes.c_uint8 * (n * dtype.itemsize)).from_address(cur[0])
        return np.frombuffer(raw, dtype=dtype, count=n)

    def fetch(self, pinned: bool = False):
        """-> (key_rows, pair_rows) of the last build as structured numpy arrays.

        ``pinned=True`` returns views of page-locked buffers owned by the builder (no allocation, full PCIe rate); they
        are overwritten by the next ``fetch(pinned=True)`` and die with the builder.
        """
        n_rows, n_keys = int(self.info["n_rows"]), int(self.info["n_keys"])
        if pinned:
            pair, keys = self._pinned("pairs", n_rows, PAIR_ROW_DTYPE), self._pinned("keys", n_keys, KEY_ROW_DTYPE)
        else:
            pair, keys = np.zeros(n_rows, dtype=PAIR_ROW_DTYPE), np.zeros(n_keys, dtype=KEY_ROW_DTYPE)
        self._check(self._lib.ks_copy_pair_rows(self._h, _lib.ptr(pair), len(pair), 0), "ks_copy_pair_rows")
        self._check(self._lib.ks_copy_key_rows(self._h, _lib.ptr(keys), len(keys), 0), "ks_copy_key_rows")
        return keys, pair

    def build(self, records, n=None, time_ordered: bool = False, key_type: bool = False, pinned: bool = False):
        self.build_device(records, n, time_ordered, key_type)
        return self.fetch(pinned)

    def pinned_records(self, n: int) -> np.ndarray:
        """A page-locked record array owned by the builder: fill it and pass it to ``build`` for full-rate host-to-device copies."""
        return self._pinned("records", n, RECORD_DTYPE)

    # -- stages
    def hash_keys(self, records, key_type: bool = False) -> np.ndarray:
        rec = np.ascontiguousarray(records, dtype=RECORD_DTYPE)
        out = np.zeros(len(rec), dtype=np.uint64)
        self._check(self._lib.ks_hash_keys(self._h, _lib.ptr(rec), len(rec), _lib.KEY_TYPE if key_type else 0, _lib.ptr(out)), "ks_hash_keys")
        return out

    def sort_pairs(self, keys: np.ndarray, vals: np.ndarray | None = None, begin_bit: int = 0, end_bit: int | None = None):
        """Stable radix sort on key bits [begin_bit, end_bit); returns sorted copies."""
        keys = np.array(keys, copy=True)
        fn = {np.dtype(np.uint64): self._lib.ks_sort_pairs_u64, np.dtype(np.uint32): self._lib.ks_sort_pairs_u32}[keys.dtype]
        if vals is not None:
            vals = np.array(vals, dtype=keys.dtype, copy=True)
        end_bit = keys.dtype.itemsize * 8 if end_bit is None else end_bit
        self._check(fn(self._h, _lib.ptr(keys), _lib.ptr(vals), len(keys), begin_bit, end_bit, 0), "ks_sort_pairs")
        return keys, vals

    def sort_launches(self, records, key_type: bool = False):
        rec = np.ascontiguousarray(records, dtype=RECORD_DTYPE)
        keys = np.zeros(len(rec), dtype=np.uint64)
        start = np.zeros(len(rec), dtype=np.uint64)
        self._check(
            self._lib.ks_sort_launches(self._h, _lib.ptr(rec), len(rec), _lib.KEY_TYPE if key_type else 0, _lib.ptr(keys), _lib.ptr(start)),
            "ks_sort_launches",
        )
        return keys, start

    def join_overlaps(self, records):
        """-> (idx_a, idx_b): positions, in the start_ns-ordered trace, of every overlapping launch pair."""
        rec = np.ascontiguousarray(records, dtype=RECORD_DTYPE)
        cnt = self._check(self._lib.ks_join_overlaps(self._h, _lib.ptr(rec), len(rec), 0, None, None, 0), "ks_join_overlaps")
        ia = np.zeros(max(cnt, 1), dtype=np.uint32)
        ib = np.zeros(max(cnt, 1), dtype=np.uint32)
        cnt2 = self._check(self._lib.ks_join_overlaps(self._h, _lib.ptr(rec), len(rec), 0, _lib.ptr(ia), _lib.ptr(ib), len(ia)), "ks_join_overlaps")
        assert cnt2 == cnt
        return ia[:cnt], ib[:cnt]

    def segment_stats(self, values: np.ndarray, offsets: np.ndarray) -> np.ndarray:
        """-> (n_segments, 6) uint64: count, sum, min, max, x[(n-1)//2], x[n//2] per segment."""
        values = np.ascontiguousarray(values, dtype=np.uint32)
        offsets = np.ascontiguousarray(offsets, dtype=np.uint64)
        nseg = len(offsets) - 1
        out = np.zeros((max(nseg, 0), 6), dtype=np.uint64)
        self._check(self._lib.ks_segment_stats(self._h, _lib.ptr(values), _lib.ptr(offsets), nseg, 0, _lib.ptr(out)), "ks_segment_stats")
        return out

    def segment_hist(self, values: np.ndarray, offsets: np.ndarray, n_bins: int, log2_bins: bool = False) -> np.ndarray:
        """-> (n_segments, n_bins) uint32: per segment a histogram of its values (bin = value, or its bit length; clamped)."""
        values = np.ascontiguousarray(values, dtype=np.uint32)
        offsets = np.ascontiguousarray(offsets, dtype=np.uint64)
        nseg = len(offsets) - 1
        out = np.zeros((max(nseg, 0), n_bins), dtype=np.uint32)
        self._check(self._lib.ks_segment_hist(self._h, _lib.ptr(values), _lib.ptr(offsets), nseg, n_bins, int(log2_bins), 0, _lib.ptr(out)), "ks_segment_hist")
        return out

    def tsv_extract(self, text, columns) -> list:
        """Columns of a tab-separated log with a header line, parsed on the device.  ``text``: bytes or a uint8 array;
        ``columns``: [(column index, kind)] with kind one of ``_lib.COL_*``.  -> one uint64 array per requested column
        (all ones where a field is blank or malformed)."""
        text = np.frombuffer(text, dtype=np.uint8) if isinstance(text, (bytes, bytearray, memoryview)) else np.ascontiguousarray(text, dtype=np.uint8)
        cols = (ctypes.c_uint32 * len(columns))(*[int(c) for c, _ in columns])
        kinds = (ctypes.c_uint32 * len(columns))(*[int(k) for _, k in columns])
        cap = max(int(np.count_nonzero(text == 10)) + 1, 1)  # at least as many as there are lines
        out = np.zeros((len(columns), cap), dtype=np.uint64)
        rows = self._check(self._lib.ks_tsv_extract(self._h, _lib.ptr(text), len(text), len(columns), cols, kinds, _lib.ptr(out), cap, 0), "ks_tsv_extract")
        return [out[i, :rows].copy() for i in range(len(columns))]

    def count_batches(self, start1, start2):
        """[n_alone, n_pairs] of scheduler/postprocess.py:17-41 (the caller slices file 1 to its last 200,000 rows)."""
        s1 = np.ascontiguousarray(start1, dtype=np.uint64)
        s2 = np.ascontiguousarray(start2, dtype=np.uint64)
        out = (ctypes.c_uint64 * 2)()
        self._check(self._lib.ks_count_batches(self._h, _lib.ptr(s1), len(s1), _lib.ptr(s2), len(s2), 0, out), "ks_count_batches")
        return [int(out[0]), int(out[1])]

    def combine_duplicates(self, group: np.ndarray, launches: np.ndarray, values: np.ndarray, n_groups: int):
        group = np.ascontiguousarray(group, dtype=np.uint32)
        launches = np.ascontiguousarray(launches, dtype=np.float64)
        values = np.ascontiguousarray(values, dtype=np.float64).reshape(len(group), -1)
        cols = values.shape[1]
        total = np.zeros(n_groups, dtype=np.float64)
        means = np.zeros((n_groups, cols), dtype=np.float64)
        self._check(
            self._lib.ks_combine_duplicates(self._h, _lib.ptr(group), _lib.ptr(launches), _lib.ptr(values), len(group), cols, n_groups, 0,
                                            _lib.ptr(total), _lib.ptr(means)),
            "ks_combine_duplicates",
        )
        return total, means

    def pool_launches(self, group: np.ndarray, values: np.ndarray, n_groups: int):
        """-> (launches [n_groups] uint64, mean [n_groups, cols], sample std [n_groups, cols]); NaN cells are absent values."""
        group = np.ascontiguousarray(group, dtype=np.uint32)
        values = np.ascontiguousarray(values, dtype=np.float64).reshape(len(group), -1)
        cols = values.shape[1]
        launches = np.zeros(n_groups, dtype=np.uint64)
        mean = np.zeros((n_groups, cols), dtype=np.float64)
        std = np.zeros((n_groups, cols), dtype=np.float64)
        self._check(
            self._lib.ks_pool_launches(self._h, _lib.ptr(group), _lib.ptr(values), len(group), cols, n_groups, 0, _lib.ptr(launches), _lib.ptr(mean), _lib.ptr(std)),
            "ks_pool_launches",
        )
        return launches, mean, std

    # -- the resident table: windows of new launches merged into statistics that stay on the device
    def update_begin(self, key_type: bool = False) -> None:
        """Starts an empty resident table on this builder (at most 2,048 distinct keys; the builder belongs to the session
        until ``update_end``)."""
        self._check(self._lib.ks_update_begin(self._h, _lib.KEY_TYPE if key_type else 0), "ks_update_begin")

    def update(self, records, n=None) -> int:
        """Merges one window of launches (start order, not earlier than the previous window); returns the samples merged.
        ``self.update_info`` holds the window's counts and the device time of the update (``ms_total``)."""
        arg = self._records_arg(records, n)
        info = _lib.KsTableInfo()
        r = self._check(self._lib.ks_update(self._h, arg[0], arg[1], arg[2], ctypes.byref(info)), "ks_update")
        self.update_info = info.as_dict()
        return r

    def update_table(self):
        """-> (key_rows, pair_rows): exactly the table ``build`` gives for all launches merged so far."""
        rows = self._check(self._lib.ks_update_table(self._h), "ks_update_table")
        keys = np.zeros(2048, dtype=KEY_ROW_DTYPE)  # the most keys a session holds
        nk = self._check(self._lib.ks_copy_key_rows(self._h, _lib.ptr(keys), len(keys), 0), "ks_copy_key_rows")
        pairs = np.zeros(rows, dtype=PAIR_ROW_DTYPE)
        self._check(self._lib.ks_copy_pair_rows(self._h, _lib.ptr(pairs), len(pairs), 0), "ks_copy_pair_rows")
        self.info = {"n_rows": rows, "n_keys": nk}
        return keys[:nk].copy(), pairs

    def update_end(self) -> None:
        self._lib.ks_update_end(self._h)
