"""Seeded synthetic launch traces with the shapes of the benchmark configurations.

Real traces come from the interception agent (reference: scheduler/agent.cpp:643-709) while two or more
model servers share a GPU; they need model weights and request datasets that are not available offline, so
the benchmark and the tests use synthetic traces whose statistics follow the configurations:

  * every tenant is one process with at most one launch in flight (scheduler_daemon.cpp:163-166), so its
    intervals do not overlap each other; idle gaps between consecutive launches are exponential, sized for
    the configuration's utilisation (the open-loop Poisson arrivals of scheduler/online_client.py:122-131);
  * kernel keys are drawn per tenant from a Zipf law; every key has its own typical duration drawn from the
    configuration's lognormal, every launch jitters around it, and co-run launches are slowed a little;
  * the solo launches (pairprof_daemon.cpp:46 ``PAIRPROF_SOLO``) form a phase of their own before the co-run
    phase, one kernel at a time over all tenants.

The trace is returned merged and ordered by ``start_ns``.  ``interleave_solo=True`` scatters the solo launches
through the co-run phase instead (a stress case for the join's filtering, not a benchmark shape).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from .records import RECORD_DTYPE, pack_records


@dataclass
class TenantSpec:
    n_keys: int
    dur_median_ns: float
    dur_sigma: float
    utilisation: float
    grid_range: tuple = (1, 4096)
    block_choices: tuple = (64, 128, 256, 512, 1024)
    zipf_s: float = 1.0
    weight: float = 1.0  # relative wall-clock share; all tenants span the same time range


@dataclass
class TraceSpec:
    name: str
    n_records: int
    tenants: list = field(default_factory=list)
    solo_fraction: float = 0.1
    seed: int = 1
    t0_ns: int = 1_000_000_000_000  # CLOCK_MONOTONIC of a machine up for ~17 min
    corun_slowdown: float = 0.25  # co-run launches take 1 + |N(0, this)| times their solo duration
    launch_jitter_sigma: float = 0.08


def config(name: str, n_records: int | None = None, seed: int | None = None) -> TraceSpec:
    """The benchmark configurations, optionally scaled to another record count."""
    name = name.lower()
    if name == "c1":
        spec = TraceSpec("c1", 200_000, [TenantSpec(150, 20e3, 1.0, 0.6, zipf_s=1.1) for _ in range(2)], 0.30, 101)
    elif name == "c2":
        spec = TraceSpec(
            "c2",
            10_000_000,
            [
                TenantSpec(1200, 8e3, 0.6, 0.60, grid_range=(1, 132), block_choices=(128, 192, 256)),
                TenantSpec(800, 150e3, 0.6, 0.45, grid_range=(1024, 16384), block_choices=(128, 256, 512)),
            ],
            0.10,
            202,
        )
    elif name == "c3":
        spec = TraceSpec("c3", 100_000_000, [TenantSpec(1250, 12e3, 1.3, 0.8) for _ in range(4)], 0.10, 303)
    elif name == "c4":
        spec = TraceSpec("c4", 1_000_000_000, [TenantSpec(2500, 15e3, 1.0, 0.5, zipf_s=0.9) for _ in range(8)], 0.10, 404)
    elif name == "c5":
        spec = config("c2")
        spec.name, spec.n_records, spec.seed = "c5", 65_536, 505
    else:
        raise ValueError(f"unknown configuration {name!r}")
    if n_records is not None:
        spec.n_records = int(n_records)
    if seed is not None:
        spec.seed = int(seed)
    return spec


def _zipf_choice(rng, n_keys, s, size):
    p = 1.0 / np.arange(1, n_keys + 1) ** s
    cdf = np.cumsum(p / p.sum())
    return np.minimum(np.searchsorted(cdf, rng.random(size)), n_keys - 1)


def generate(spec: TraceSpec, interleave_solo: bool = False, window: int = 0) -> np.ndarray:
    """-> records (RECORD_DTYPE), ordered by start_ns.

    ``window`` selects an independent stretch of the same workload: the key tables (names, grids, typical durations)
    depend on ``spec.seed`` only, the launches on (seed, window).  Multi-GPU runs give every rank its own window.
    """
    key_rng = np.random.default_rng(spec.seed)
    rng = np.random.default_rng([spec.seed, 7919 + window])
    nt = len(spec.tenants)
    # launches per tenant: equal wall-clock span => count ~ utilisation / mean duration
    mean_dur = np.array([t.dur_median_ns * np.exp(0.5 * t.dur_sigma**2) for t in spec.tenants])
    rate = np.array([t.utilisation * t.weight for t in spec.tenants]) / mean_dur
    n_per = np.maximum((spec.n_records * rate / rate.sum()).astype(np.int64), 1)
    n_per[0] += spec.n_records - n_per.sum()
    assert (n_per > 0).all()

    cols = {k: [] for k in ("name_id", "grid", "block", "smem", "tenant", "solo", "start", "dur")}
    name_base = 0
    for t, (ts, n) in enumerate(zip(spec.tenants, n_per)):
        n = int(n)
        k = ts.n_keys
        key_name = name_base + key_rng.permutation(k).astype(np.uint32)
        name_base += k
        key_grid = np.stack([key_rng.integers(ts.grid_range[0], ts.grid_range[1] + 1, k), key_rng.integers(1, 3, k), np.ones(k, np.int64)], axis=1)
        key_block = np.stack([key_rng.choice(ts.block_choices, k), np.ones(k, np.int64), np.ones(k, np.int64)], axis=1)
        key_smem = key_rng.choice([0, 0, 0, 16384, 49152, 98304], k)
        key_dur = ts.dur_median_ns * np.exp(ts.dur_sigma * key_rng.standard_normal(k))
        kix = _zipf_choice(rng, k, ts.zipf_s, n)
        solo = rng.random(n) < spec.solo_fraction
        d = key_dur[kix] * np.exp(spec.launch_jitter_sigma * rng.standard_normal(n))
        d = np.where(solo, d, d * (1.0 + np.abs(spec.corun_slowdown * rng.standard_normal(n))))
        d = np.clip(np.rint(d), 200, 2**31 - 1).astype(np.int64)
        cols["name_id"].append(key_name[kix])
        cols["grid"].append(key_grid[kix])
        cols["block"].append(key_block[kix])
        cols["smem"].append(key_smem[kix])
        cols["tenant"].append(np.full(n, t, np.int64))
        cols["solo"].append(solo)
        cols["dur"].append(d)
        # co-run timeline of this tenant: gap, launch, gap, launch ...  (gap mean gives the utilisation)
        gap_mean = mean_dur[t] * (1.0 - ts.utilisation) / ts.utilisation
        gaps = np.rint(rng.exponential(gap_mean, n)).astype(np.int64) + 1
        if interleave_solo:
            st = np.cumsum(gaps + d) - d
        else:
            step = np.where(solo, 0, gaps + d)
            st = np.cumsum(step) - np.where(solo, 0, d)
        cols["start"].append(st)

    cat = {k: np.concatenate(v) for k, v in cols.items()}
    solo = cat["solo"]
    start = cat["start"].astype(np.int64)
    if not interleave_solo:
        # solo phase: every solo launch of every tenant back to back (shuffled), then the co-run phase
        sidx = np.flatnonzero(solo)
        sidx = sidx[rng.permutation(len(sidx))]
        sd = cat["dur"][sidx] + 500
        sstart = np.cumsum(sd) - sd
        start[sidx] = sstart
        phase2 = int(sd.sum()) + 1_000_000
        start[~solo] += phase2
    start = start + spec.t0_ns
    end = start + cat["dur"]
    order = np.argsort(start, kind="stable")
    rec = pack_records(cat["name_id"], cat["grid"], cat["block"], cat["smem"], cat["tenant"], solo, start, end)
    return np.ascontiguousarray(rec[order])


def _key_tables(spec: TraceSpec):
    """Per tenant the launch shapes, typical durations and Zipf table of its keys: a function of ``spec.seed`` only."""
    key_rng = np.random.default_rng(spec.seed)
    tables, name_base = [], 0
    for ts in spec.tenants:
        k = ts.n_keys
        name = (name_base + key_rng.permutation(k)).astype(np.uint32)
        name_base += k
        grid = np.stack([key_rng.integers(ts.grid_range[0], ts.grid_range[1] + 1, k), key_rng.integers(1, 3, k), np.ones(k, np.int64)], axis=1).astype(np.uint32)
        block = np.stack([key_rng.choice(ts.block_choices, k), np.ones(k, np.int64), np.ones(k, np.int64)], axis=1).astype(np.uint32)
        smem = key_rng.choice([0, 0, 0, 16384, 49152, 98304], k).astype(np.uint32)
        dur = (ts.dur_median_ns * np.exp(ts.dur_sigma * key_rng.standard_normal(k))).astype(np.float64)
        p = 1.0 / np.arange(1, k + 1) ** ts.zipf_s
        cdf = np.cumsum(p / p.sum())
        cdf[-1] = 1.0
        tables.append(tuple(np.ascontiguousarray(a) for a in (name, grid, block, smem, dur, cdf)))
    return tables


def generate_fast(spec: TraceSpec, window: int = 0, out: np.ndarray | None = None, threads: int = 0, interleave_solo: bool = False) -> np.ndarray:
    """The same workload model as ``generate`` from the library's multi-threaded host generator (``ks_synth_trace``):
    traces of 10^8 launches in seconds.  The launches differ from ``generate``'s (another random stream); the key tables
    are the same.  ``out``: a record buffer to fill (e.g. pinned memory), else a new array.  ``interleave_solo``: the solo
    launches take their turn on their tenant's timeline (the online configuration) instead of a phase of their own in front.
    -> records, ordered by start_ns.
    """
    from . import _lib

    lib = _lib.load()
    mean_dur = np.array([t.dur_median_ns * np.exp(0.5 * t.dur_sigma**2) for t in spec.tenants])
    rate = np.array([t.utilisation * t.weight for t in spec.tenants]) / mean_dur
    n_per = np.maximum((spec.n_records * rate / rate.sum()).astype(np.int64), 1)
    n_per[0] += spec.n_records - n_per.sum()
    assert (n_per > 0).all()
    tables = _key_tables(spec)
    arr = (_lib.KsSynthTenant * len(spec.tenants))()
    for t, (ts, tab) in enumerate(zip(spec.tenants, tables)):
        name, grid, block, smem, dur, cdf = tab
        arr[t].n_keys, arr[t].tenant, arr[t].n_launches = ts.n_keys, t, int(n_per[t])
        arr[t].name_id, arr[t].grid, arr[t].block, arr[t].smem = name.ctypes.data, grid.ctypes.data, block.ctypes.data, smem.ctypes.data
        arr[t].dur_ns, arr[t].cdf = dur.ctypes.data, cdf.ctypes.data
        arr[t].gap_mean_ns = float(mean_dur[t] * (1.0 - ts.utilisation) / ts.utilisation)
    if out is None:
        out = np.empty(spec.n_records, dtype=RECORD_DTYPE)
    assert out.dtype == RECORD_DTYPE and len(out) >= spec.n_records and out.flags["C_CONTIGUOUS"]
    seed = (int(spec.seed) << 20) ^ (7919 + int(window))
    r = lib.ks_synth_trace(arr, len(spec.tenants), spec.solo_fraction, spec.launch_jitter_sigma, spec.corun_slowdown, seed, spec.t0_ns,
                           out.ctypes.data, len(out), threads, 1 if interleave_solo else 0)
    if r < 0:
        raise _lib.KsError(int(-r), "ks_synth_trace")
    return out[: int(r)]


def shuffled(records: np.ndarray, seed: int = 7) -> np.ndarray:
    """The same launches in random order (exercises the time sort in front of the join)."""
    rng = np.random.default_rng(seed)
    return np.ascontiguousarray(records[rng.permutation(len(records))])


def to_dtype(buf) -> np.ndarray:
    return np.frombuffer(buf, dtype=RECORD_DTYPE)
