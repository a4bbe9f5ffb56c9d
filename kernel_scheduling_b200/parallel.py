"""Multi-GPU trace -> interference-table path: one process per GPU, each owning one window of the trace.

The start-ordered trace is cut into ``world`` windows by record position.  The steps, with the collective between
them (NCCL through ``torch.distributed`` on GPUs):

  1. K1 over the own window; pick the launches that are still running at the window's last start (``tail``)
  2. all-gather of the tails  -> rank r decodes rank r-1's tail as its halo (a pair of overlapping launches is
     PRODUCED by the rank that owns its later launch, so every pair is produced exactly once)
  3. all-gather of the distinct keys -> every dictionary holds every key -> identical dense key ids on every rank
  4. sum of the per-key launch counts
  5. solo samples + K3 join; coarse histogram of the samples' sort keys; sum -> splitters that cut the key space
     into ``world`` ranges of about equal sample count (a whole table row always lands on one rank)
  6. partition by destination; all-to-all of the samples (samples travel, not partial tables: the median is exact)
  7. K2 sort + K4 statistics of the received range; max-merge of the solo times (each key's solo row lives on
     exactly one rank); tables
  8. all-gather of the table shards: ranges are ordered, so their concatenation in rank order is the sorted table

``build_steps`` is a generator: it yields one request per collective and is driven either by ``run_distributed``
(torch.distributed, one process per rank) or by ``run_in_process`` (all ranks in one process, one after the other;
used to check the multi-rank logic on a single GPU and on the CPU).  The per-rank compute is behind a ``stages``
object: ``GpuStages`` (the C ABI of libks_b200.so) in production.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import _lib
from .records import KEY_ROW_DTYPE, PAIR_ROW_DTYPE, RECORD_DTYPE

HALO_MAX = 4096
HIST_BINS = 4096


def choose_splitters(hist: np.ndarray, world: int) -> list[int]:
    """First histogram bin of ranks 1 .. world-1 so that every rank gets about total / world samples.

    A rank's range is [splitter[r-1], splitter[r]) in bins; a bin is never split, so all samples of a sort key (one
    table row) share a destination.  Splitters are non-decreasing; an empty range is legal.
    """
    hist = np.asarray(hist, dtype=np.int64)
    total = int(hist.sum())
    before = np.concatenate([[0], np.cumsum(hist)[:-1]])  # samples in front of each bin
    out = []
    for r in range(1, world):
        target = (total * r + world - 1) // world
        b = int(np.searchsorted(before, target, side="left"))
        out.append(min(b, len(hist)))
    return out


def build_steps(stages, rank: int, world: int, key_type: bool = False, on_device: bool = False):
    """Generator over the collectives of one rank; returns (key_rows, pair_rows) of the WHOLE table as numpy arrays
    (``on_device``: as uint8 tensors on the stages' device, no copy to the host)."""
    stages.begin(key_type)
    # -- halo
    tail = stages.tail()  # uint8 tensor, 48 bytes per record, start order
    padded = stages.zeros((HALO_MAX * 48 + 8,), torch.uint8)
    padded[: tail.numel()] = tail
    padded[HALO_MAX * 48:] = torch.tensor(list(int(tail.numel() // 48).to_bytes(8, "little")), dtype=torch.uint8, device=padded.device)
    tails = yield ("all_gather", padded)
    # the halo of rank r: launches of ANY earlier window that are still running when window r begins (a launch can span
    # several windows); every rank holds every tail after the all-gather, the filter runs on the host (a few KB)
    first = stages.first_start()
    parts = []
    for q in range(rank):
        t = tails[q].cpu().numpy()
        n_q = int.from_bytes(t[HALO_MAX * 48:].tobytes(), "little")
        recs = np.frombuffer(t[: n_q * 48].tobytes(), dtype=RECORD_DTYPE)
        if first is not None:
            parts.append(recs[recs["end_ns"] > np.uint64(first)])
    halo = np.concatenate(parts) if parts else np.zeros(0, dtype=RECORD_DTYPE)
    if len(halo) > HALO_MAX:
        raise _lib.KsError(_lib.ERR_CAPACITY, f"{len(halo)} launches of earlier windows reach into window {rank}; the halo holds {HALO_MAX}")
    stages.halo(stages.from_bytes(halo.tobytes()))
    # -- global keys
    keys, words = stages.local_keys()  # int64 [k], uint8 [k * 32]
    counts = yield ("all_gather", stages.tensor([keys.numel()], torch.int64))
    kmax = max(int(c[0]) for c in counts)
    kp = stages.zeros((kmax,), torch.int64)
    wp = stages.zeros((kmax * 32,), torch.uint8)
    kp[: keys.numel()] = keys
    wp[: words.numel()] = words
    all_k = yield ("all_gather", kp)
    all_w = yield ("all_gather", wp)
    n_keys = stages.global_keys(torch.cat(all_k), torch.cat(all_w))  # zero keys (padding) are skipped by the insert
    launches, solo = stages.counts_export()
    launches = yield ("all_reduce_sum", launches)
    solo = yield ("all_reduce_sum", solo)
    stages.counts_import(launches, solo)
    # -- samples, splitters, exchange
    stages.samples()
    hist, shift = stages.key_histogram()
    hist = yield ("all_reduce_sum", hist)
    splitters = choose_splitters(hist.cpu().numpy(), world)
    send, send_counts = stages.partition(splitters, shift, world)  # int32 [n, 4] grouped by destination
    recv = yield ("all_to_all", send, send_counts)
    stages.reduce(recv)
    # -- solo times: each key's solo row was reduced by exactly one rank
    solo_ns = stages.solo_export()
    neg = torch.where(torch.isnan(solo_ns), torch.full_like(solo_ns, float("-inf")), solo_ns)
    neg = yield ("all_reduce_max", neg)
    stages.solo_import(torch.where(torch.isinf(neg) & (neg < 0), torch.full_like(neg, float("nan")), neg))
    stages.finalize()
    key_rows, pair_rows = stages.tables()  # uint8 tensors: this rank's key range
    # -- the whole table on every rank
    sizes = yield ("all_gather", stages.tensor([pair_rows.numel()], torch.int64))
    pmax = max(int(s[0]) for s in sizes)
    pp = stages.zeros((pmax,), torch.uint8)
    pp[: pair_rows.numel()] = pair_rows
    shards = yield ("all_gather", pp)
    table = torch.cat([sh[: int(sz[0])] for sh, sz in zip(shards, sizes)])
    if on_device:
        return key_rows, table
    return (np.frombuffer(key_rows.cpu().numpy().tobytes(), dtype=KEY_ROW_DTYPE)[:n_keys].copy(),
            np.frombuffer(table.cpu().numpy().tobytes(), dtype=PAIR_ROW_DTYPE).copy())


# ---------------------------------------------------------------------------------------------------------------
def run_distributed(gen, group=None):
    """Drives one rank's generator with torch.distributed collectives (NCCL on GPUs, gloo on CPU tensors)."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    try:
        req = next(gen)
        while True:
            kind = req[0]
            if kind == "all_gather":
                out = [torch.empty_like(req[1]) for _ in range(world)]
                dist.all_gather(out, req[1].contiguous(), group=group)
                res = out
            elif kind == "all_reduce_sum":
                res = req[1].clone()
                dist.all_reduce(res, op=dist.ReduceOp.SUM, group=group)
            elif kind == "all_reduce_max":
                res = req[1].clone()
                dist.all_reduce(res, op=dist.ReduceOp.MAX, group=group)
            elif kind == "all_to_all":
                send, counts = req[1], [int(c) for c in req[2]]
                ct = torch.tensor(counts, dtype=torch.int64, device=send.device)
                rc = torch.empty_like(ct)
                dist.all_to_all_single(rc, ct, group=group)
                rcounts = [int(c) for c in rc.cpu().tolist()]
                res = torch.empty((sum(rcounts), send.shape[1]), dtype=send.dtype, device=send.device)
                dist.all_to_all_single(res, send.contiguous(), output_split_sizes=rcounts, input_split_sizes=counts, group=group)
            else:
                raise ValueError(kind)
            req = gen.send(res)
    except StopIteration as stop:
        return stop.value


def run_in_process(gens):
    """Drives the generators of all ranks in one process, fulfilling each collective locally."""
    world = len(gens)
    reqs, results, done = [None] * world, [None] * world, [False] * world
    for r, g in enumerate(gens):
        reqs[r] = next(g)
    while not all(done):
        kind = reqs[0][0]
        assert all(q[0] == kind for q in reqs), "ranks disagree on the next collective"
        if kind == "all_gather":
            res = [[q[1].clone() for q in reqs] for _ in range(world)]
        elif kind == "all_reduce_sum":
            tot = sum(q[1] for q in reqs)
            res = [tot.clone() for _ in range(world)]
        elif kind == "all_reduce_max":
            tot = reqs[0][1]
            for q in reqs[1:]:
                tot = torch.maximum(tot, q[1])
            res = [tot.clone() for _ in range(world)]
        elif kind == "all_to_all":
            res = []
            offs = [np.concatenate([[0], np.cumsum([int(c) for c in q[2]])]) for q in reqs]
            for dst in range(world):
                res.append(torch.cat([reqs[src][1][int(offs[src][dst]): int(offs[src][dst + 1])] for src in range(world)]))
        else:
            raise ValueError(kind)
        for r, g in enumerate(gens):
            try:
                reqs[r] = g.send(res[r])
            except StopIteration as stop:
                results[r], done[r] = stop.value, True
        assert all(done) or not any(done), "ranks finished at different steps"
    return results


# ---------------------------------------------------------------------------------------------------------------
class GpuStages:
    """One rank's compute through the C ABI (ks_mg_*).  ``records`` is a uint8 CUDA tensor of 48-byte records."""

    def __init__(self, builder, records: torch.Tensor):
        self.b = builder
        self.lib = builder._lib
        self.h = builder._h
        self.records = records
        self.device = records.device
        self.n_owned = records.numel() // 48
        self.n_keys = 0
        self._keep = []

    # tensors
    def zeros(self, shape, dtype):
        return torch.zeros(shape, dtype=dtype, device=self.device)

    def tensor(self, data, dtype):
        return torch.tensor(data, dtype=dtype, device=self.device)

    def from_bytes(self, raw: bytes):
        return torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(self.device) if raw else self.zeros((0,), torch.uint8)

    def first_start(self):
        """start_ns of the window's first record, or None for an empty window."""
        if self.n_owned == 0:
            return None
        return int(np.frombuffer(self.records[:48].cpu().numpy().tobytes(), dtype=RECORD_DTYPE)["start_ns"][0])

    def _ck(self, r, what):
        return self.b._check(r, what)

    @staticmethod
    def _p(t):
        return ctypes.c_void_p(t.data_ptr()) if t.numel() else None

    # phases
    def begin(self, key_type):
        self._ck(self.lib.ks_mg_begin(self.h, self._p(self.records), self.n_owned, _lib.KEY_TYPE if key_type else 0), "ks_mg_begin")

    def tail(self):
        out = self.zeros((HALO_MAX * 48,), torch.uint8)
        n = self._ck(self.lib.ks_mg_tail(self.h, self._p(out), HALO_MAX), "ks_mg_tail")
        return out[: n * 48]

    def halo(self, rec):
        self._keep.append(rec)
        self._ck(self.lib.ks_mg_halo(self.h, self._p(rec), rec.numel() // 48), "ks_mg_halo")

    def local_keys(self):
        keys = self.zeros((65536,), torch.int64)
        words = self.zeros((65536 * 32,), torch.uint8)
        n = self._ck(self.lib.ks_mg_local_keys(self.h, self._p(keys), self._p(words), 65536), "ks_mg_local_keys")
        return keys[:n], words[: n * 32]

    def global_keys(self, keys, words):
        keys, words = keys.contiguous(), words.contiguous()
        self.n_keys = self._ck(self.lib.ks_mg_global_keys(self.h, self._p(keys), self._p(words), keys.numel()), "ks_mg_global_keys")
        return self.n_keys

    def counts_export(self):
        a, b = self.zeros((self.n_keys,), torch.int64), self.zeros((self.n_keys,), torch.int64)
        self._ck(self.lib.ks_mg_counts(self.h, ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(b.data_ptr()), 0), "ks_mg_counts")
        return a, b

    def counts_import(self, a, b):
        a, b = a.contiguous(), b.contiguous()
        self._ck(self.lib.ks_mg_counts(self.h, ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(b.data_ptr()), 1), "ks_mg_counts")

    def samples(self):
        self.n_samples = self._ck(self.lib.ks_mg_samples(self.h), "ks_mg_samples")
        return self.n_samples

    def key_histogram(self):
        hist = self.zeros((HIST_BINS,), torch.int64)
        shift = ctypes.c_uint32(0)
        self._ck(self.lib.ks_mg_key_histogram(self.h, ctypes.c_void_p(hist.data_ptr()), ctypes.byref(shift)), "ks_mg_key_histogram")
        return hist, int(shift.value)

    def partition(self, splitters, shift, world):
        send = torch.empty((max(self.n_samples, 1), 4), dtype=torch.int32, device=self.device)
        sp = (ctypes.c_uint32 * max(len(splitters), 1))(*splitters)
        counts = (ctypes.c_uint64 * world)()
        self._ck(self.lib.ks_mg_partition(self.h, sp, shift, world, ctypes.c_void_p(send.data_ptr()), send.shape[0], counts), "ks_mg_partition")
        return send[: self.n_samples], [int(c) for c in counts]

    def reduce(self, recv):
        recv = recv.contiguous()
        self._keep.append(recv)
        self._ck(self.lib.ks_mg_reduce(self.h, self._p(recv), recv.shape[0]), "ks_mg_reduce")

    def solo_export(self):
        t = self.zeros((self.n_keys,), torch.float64)
        if self.n_keys:
            self._ck(self.lib.ks_mg_solo(self.h, ctypes.c_void_p(t.data_ptr()), 0), "ks_mg_solo")
        return t

    def solo_import(self, t):
        t = t.contiguous()
        if self.n_keys:
            self._ck(self.lib.ks_mg_solo(self.h, ctypes.c_void_p(t.data_ptr()), 1), "ks_mg_solo")

    def finalize(self):
        self.n_rows = self._ck(self.lib.ks_mg_finalize(self.h), "ks_mg_finalize")
        return self.n_rows

    def tables(self):
        keys = self.zeros((max(self.n_keys, 1) * KEY_ROW_DTYPE.itemsize,), torch.uint8)
        pairs = self.zeros((max(self.n_rows, 1) * PAIR_ROW_DTYPE.itemsize,), torch.uint8)
        self._ck(self.lib.ks_copy_key_rows(self.h, ctypes.c_void_p(keys.data_ptr()), max(self.n_keys, 1), _lib.ON_DEVICE), "ks_copy_key_rows")
        self._ck(self.lib.ks_copy_pair_rows(self.h, ctypes.c_void_p(pairs.data_ptr()), max(self.n_rows, 1), _lib.ON_DEVICE), "ks_copy_pair_rows")
        self._keep.clear()
        return keys[: self.n_keys * KEY_ROW_DTYPE.itemsize], pairs[: self.n_rows * PAIR_ROW_DTYPE.itemsize]


def split_windows(n_records: int, world: int) -> list[tuple[int, int]]:
    """Record ranges [lo, hi) of the windows: equal record counts, the remainder to the first windows."""
    base, extra = divmod(n_records, world)
    out, lo = [], 0
    for r in range(world):
        hi = lo + base + (1 if r < extra else 0)
        out.append((lo, hi))
        lo = hi
    return out
