"""Multi-GPU trace -> interference-table path: one process per GPU, each owning one window of the trace.

The start-ordered trace is cut into ``world`` windows by record position.  The steps, with the collective between
them (NCCL through ``torch.distributed`` on GPUs):

  1. K1 over the own window; pick the launches that are still running at the window's last start (``tail``)
  2. all-gather of [tails | distinct keys]: every dictionary then holds every key -> identical dense key ids on
     every rank; rank r decodes the earlier ranks' tails that reach into its window as its halo (a pair of
     overlapping launches is PRODUCED by the rank that owns its later launch: exactly once)
  3. solo samples + K3 join; all-gather of [coarse histogram of the samples' sort keys | per-key launch counts]
     -> splitters that cut the key space into ``world`` ranges of about equal sample count (a whole table row
     always lands on one rank), and how many samples every rank will send to every other
  4. partition by destination; all-to-all of the samples (samples travel, not partial tables: the median is exact)
  5. K2 sort + K4 statistics of the received range; all-gather of [solo times | shard sizes] (each key's solo row
     lives on exactly one rank); tables
  6. all-gather of the table shards: ranges are ordered, so their concatenation in rank order is the sorted table

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


_key_capacity = 4096  # keys per rank that fit the first exchange; grown (on every rank alike) when a rank has more


def _u64_bytes(dev, *vals):
    return torch.frombuffer(bytearray(b"".join(int(v).to_bytes(8, "little") for v in vals)), dtype=torch.uint8).to(dev)


def _u64_at(buf_cpu: np.ndarray, i: int) -> int:
    return int.from_bytes(buf_cpu[8 * i: 8 * i + 8].tobytes(), "little")


def build_steps(stages, rank: int, world: int, key_type: bool = False, on_device: bool = False):
    """Generator over the collectives of one rank (five per table); returns (key_rows, pair_rows) of the WHOLE table as
    numpy arrays (``on_device``: as uint8 tensors on the stages' device, no copy to the host)."""
    global _key_capacity
    stages.begin(key_type)
    # -- collective 1: [n_tail, n_keys | tail records | distinct keys | their launch fields] of every rank
    tail = stages.tail()               # uint8, 48 bytes per record, start order
    keys, words = stages.local_keys()  # int64 [k], uint8 [k * 32]  (own window; halo keys arrive from their owners)
    while True:
        cap = _key_capacity
        buf = stages.zeros((16 + HALO_MAX * 48 + cap * 40,), torch.uint8)
        buf[:16] = _u64_bytes(buf.device, tail.numel() // 48, keys.numel())
        buf[16: 16 + tail.numel()] = tail
        k_fit = min(keys.numel(), cap)
        if k_fit:
            buf[16 + HALO_MAX * 48: 16 + HALO_MAX * 48 + k_fit * 8] = keys[:k_fit].contiguous().view(torch.uint8)
        buf[16 + HALO_MAX * 48 + cap * 8: 16 + HALO_MAX * 48 + cap * 8 + k_fit * 32] = words[: k_fit * 32]
        bufs = yield ("all_gather", buf)
        heads = [b[:16].cpu().numpy() for b in bufs]
        need = max(_u64_at(h, 1) for h in heads)
        if need <= cap:
            break
        _key_capacity = 1 << int(need - 1).bit_length()  # every rank sees the same headers and grows alike
    k0 = 16 + HALO_MAX * 48
    all_k = torch.cat([b[k0: k0 + _u64_at(h, 1) * 8] for b, h in zip(bufs, heads)]).contiguous().view(torch.int64)
    all_w = torch.cat([b[k0 + cap * 8: k0 + cap * 8 + _u64_at(h, 1) * 32] for b, h in zip(bufs, heads)])
    n_keys = stages.global_keys(all_k, all_w)
    # the halo of rank r: launches of ANY earlier window that are still running when window r begins (a launch can span
    # several windows); the filter runs on the host over a few KB
    first = stages.first_start()
    parts = []
    for q in range(rank):
        n_q = _u64_at(heads[q], 0)
        if n_q and first is not None:
            recs = np.frombuffer(bufs[q][16: 16 + n_q * 48].cpu().numpy().tobytes(), dtype=RECORD_DTYPE)
            parts.append(recs[recs["end_ns"] > np.uint64(first)])
    halo = np.concatenate(parts) if parts else np.zeros(0, dtype=RECORD_DTYPE)
    if len(halo) > HALO_MAX:
        raise _lib.KsError(_lib.ERR_CAPACITY, f"{len(halo)} launches of earlier windows reach into window {rank}; the halo holds {HALO_MAX}")
    stages.halo(stages.from_bytes(halo.tobytes()))
    # -- samples; collective 2: [sample-key histogram | per-key launch counts] of every rank
    launches, solo = stages.counts_export()
    stages.samples()
    hist, shift = stages.key_histogram()
    gathered = yield ("all_gather", torch.cat([hist, launches, solo]))
    hists = [g[:HIST_BINS].cpu().numpy() for g in gathered]
    total = torch.stack(gathered).sum(dim=0)
    stages.counts_import(total[HIST_BINS: HIST_BINS + n_keys].contiguous(), total[HIST_BINS + n_keys:].contiguous())
    splitters = choose_splitters(np.sum(hists, axis=0), world)
    edges = [0] + [min(x, HIST_BINS) for x in splitters] + [HIST_BINS]
    recv_counts = [int(h[edges[rank]: edges[rank + 1]].sum()) for h in hists]  # what each rank holds for my range
    # -- collective 3: the samples travel to the rank that owns their key range
    send_counts = [int(hists[rank][edges[d]: edges[d + 1]].sum()) for d in range(world)]  # what I hold for every range
    send = stages.partition(splitters, shift, world)  # int32 [n, 4] grouped by destination
    recv = yield ("all_to_all", send, send_counts, recv_counts)
    stages.reduce(recv)
    # -- collective 4: [solo times | size of the table shard]; each key's solo row was reduced by exactly one rank
    solo_ns = stages.solo_export()
    n_rows = stages.row_count()
    got = yield ("all_gather", torch.cat([solo_ns, stages.tensor([float(n_rows)], torch.float64)]))
    stacked = torch.stack([g[:n_keys] for g in got])
    merged = torch.where(torch.isnan(stacked), torch.full_like(stacked, float("-inf")), stacked).max(dim=0).values
    stages.solo_import(torch.where(torch.isinf(merged) & (merged < 0), torch.full_like(merged, float("nan")), merged))
    sizes = [int(g[n_keys].item()) * PAIR_ROW_DTYPE.itemsize for g in got]
    stages.finalize()
    key_rows, pair_rows = stages.tables()  # uint8 tensors: this rank's key range
    # -- collective 5: the whole table on every rank (ranges are ordered: concatenation in rank order is the sorted table)
    pp = stages.zeros((max(sizes),), torch.uint8)
    pp[: pair_rows.numel()] = pair_rows
    shards = yield ("all_gather", pp)
    table = torch.cat([sh[:sz] for sh, sz in zip(shards, sizes)])
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
                send, counts, rcounts = req[1], [int(c) for c in req[2]], [int(c) for c in req[3]]
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
                assert [int(c) for c in reqs[dst][3]] == [int(offs[src][dst + 1] - offs[src][dst]) for src in range(world)], "receive counts"
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

    def __init__(self, builder, records: torch.Tensor, first_start: int | None = None):
        if records.is_cuda and builder.stream != torch.cuda.current_stream(records.device).cuda_stream:
            # the collectives run on torch's current stream; the library must launch on the same one, or a collective
            # could still be writing a buffer the next phase reads
            raise ValueError("create the PairTableBuilder with stream=torch.cuda.current_stream().cuda_stream (and keep that stream current)")
        self.b = builder
        self.lib = builder._lib
        self.h = builder._h
        self.records = records
        self.device = records.device
        self.n_owned = records.numel() // 48
        self.n_keys = 0
        self._keep = []
        self._first_start = first_start  # start_ns of the first record when the caller knows it (saves a device read)

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
        if self._first_start is not None:
            return self._first_start
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
        self._ck(self.lib.ks_mg_partition(self.h, sp, shift, world, ctypes.c_void_p(send.data_ptr()), send.shape[0], None), "ks_mg_partition")
        return send[: self.n_samples]

    def solo_export(self):
        t = self.zeros((self.n_keys,), torch.float64)
        if self.n_keys:
            self._ck(self.lib.ks_mg_solo(self.h, ctypes.c_void_p(t.data_ptr()), 0), "ks_mg_solo")
        return t

    def solo_import(self, t):
        t = t.contiguous()
        if self.n_keys:
            self._ck(self.lib.ks_mg_solo(self.h, ctypes.c_void_p(t.data_ptr()), 1), "ks_mg_solo")

    def reduce(self, recv):
        recv = recv.contiguous()
        self._keep.append(recv)
        self._rows_total = self._ck(self.lib.ks_mg_reduce(self.h, self._p(recv), recv.shape[0]), "ks_mg_reduce")

    def row_count(self):
        """Pair rows of this rank's key range (known after reduce: rows minus solo rows)."""
        return self._ck(self.lib.ks_mg_row_count(self.h), "ks_mg_row_count")

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


class NativeSession:
    """One rank of the native build: ``ks_mg_build`` runs the phases AND the five exchanges inside the library (NCCL on the
    builder's stream, three host waits per table).  The production path on GPUs; ``build_steps`` is the same algorithm
    with the exchanges in Python, which also runs without NCCL (gloo, in-process).

    Creating a session is collective over the ranks: rank 0 makes the NCCL id, ``torch.distributed`` (any backend) hands
    it round.  ``world == 1`` needs no process group.
    """

    def __init__(self, builder, rank: int = 0, world: int = 1, group=None):
        self.b, self.rank, self.world = builder, rank, world
        lib = builder._lib
        ident = ctypes.create_string_buffer(128)
        if rank == 0:
            r = lib.ks_mg_unique_id(ident)
            if r < 0:
                raise _lib.KsError(int(-r), "ks_mg_unique_id: NCCL is not available")
        if world > 1:
            import torch.distributed as dist

            box = [ident.raw]
            dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
            ident = ctypes.create_string_buffer(box[0], 128)
        builder._check(lib.ks_mg_comm_init(builder._h, ident, rank, world), "ks_mg_comm_init")

    @property
    def peer_memory(self) -> bool:
        """True when the two bulk exchanges are stores into the other GPUs' memory (CUDA IPC over NVLink) from the kernels
        that produce the data; False when they are NCCL send/recv pairs (``KS_MG_NO_P2P`` set, or a GPU pair without peer
        access)."""
        return bool(self.b._lib.ks_mg_peer_memory(self.b._h))

    def build_device(self, records: torch.Tensor, key_type: bool = False, timing: bool = False) -> int:
        """Collective.  ``records``: this rank's window as a uint8 CUDA tensor (48 bytes per record, start order), ready on
        the builder's stream.  Returns the rows of the whole table, which stays on this rank's device (``builder.fetch``).
        ``timing``: wait for the call to finish and report the device time of its five phases in ``builder.info``."""
        if not records.is_cuda or records.dtype != torch.uint8 or records.numel() % 48:
            raise ValueError("records: a uint8 CUDA tensor of 48-byte records")
        info = _lib.KsTableInfo()
        p = ctypes.c_void_p(records.data_ptr()) if records.numel() else None
        flags = (_lib.KEY_TYPE if key_type else 0) | (_lib.TIMING if timing else 0)
        rows = self.b._check(self.b._lib.ks_mg_build(self.b._h, p, records.numel() // 48, flags, ctypes.byref(info)), "ks_mg_build")
        self.b.info = info.as_dict()
        return rows

    def build(self, records: torch.Tensor, key_type: bool = False, pinned: bool = False, fetch: bool = True):
        """-> (key_rows, pair_rows) of the whole table as numpy arrays.  Every rank holds the table on its device; a rank
        that passes ``fetch=False`` skips the copy to its host and gets (None, None) -- one copy per job is enough."""
        self.build_device(records, key_type)
        if not fetch:
            return None, None
        return self.b.fetch(pinned)

    def close(self):
        """Collective (in peer-memory mode every rank unmaps the others' buffers before any buffer is freed)."""
        self.b._lib.ks_mg_comm_destroy(self.b._h)


def split_windows(n_records: int, world: int) -> list[tuple[int, int]]:
    """Record ranges [lo, hi) of the windows: equal record counts, the remainder to the first windows."""
    base, extra = divmod(n_records, world)
    out, lo = [], 0
    for r in range(world):
        hi = lo + base + (1 if r < extra else 0)
        out.append((lo, hi))
        lo = hi
    return out
