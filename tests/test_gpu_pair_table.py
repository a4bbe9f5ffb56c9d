"""Parity of the CUDA path (through the C ABI) against the CPU oracle on seeded traces."""
import numpy as np
import pytest

from kernel_scheduling_b200 import trace
from kernel_scheduling_b200.records import RECORD_DTYPE, pack_records
from oracle import c_oracle as CO
from oracle import pair_table_oracle as O
from tests.helpers import assert_tables_match

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("cfg,n", [("c1", 200_000), ("c2", 400_000), ("c3", 300_000), ("c4", 300_000)])
@pytest.mark.parametrize("ordered", [True, False])
def test_pair_table_matches_oracle(builder, cfg, n, ordered):
    rec = trace.generate(trace.config(cfg, n))
    if not ordered:
        rec = trace.shuffled(rec)
    keys, pairs = builder.build(rec, time_ordered=ordered)
    okeys, opairs = O.build_pair_table(rec)
    assert_tables_match(keys, pairs, okeys, opairs)
    assert builder.info["n_pairs"] == int(opairs["count"].sum())
    assert builder.info["was_time_ordered"] == int(ordered)


def test_type_keys(builder):
    rec = trace.generate(trace.config("c1", 50_000))
    keys, pairs = builder.build(rec, time_ordered=True, key_type=True)
    okeys, opairs = O.build_pair_table(rec, key_mode=O.KEY_TYPE)
    assert_tables_match(keys, pairs, okeys, opairs)


def test_interleaved_solo_and_missing_baselines(builder):
    spec = trace.config("c1", 60_000)
    spec.solo_fraction = 0.02  # many keys end up without a solo launch: NaN sides
    rec = trace.generate(spec, interleave_solo=True)
    keys, pairs = builder.build(rec, time_ordered=True)
    okeys, opairs = O.build_pair_table(rec)
    assert (opairs["flags"] != 3).any() and (opairs["flags"] == 3).any()
    assert_tables_match(keys, pairs, okeys, opairs)


@pytest.mark.parametrize("n", [0, 1, 2, 31, 32, 33, 255, 256, 257, 1023, 1024, 1025, 2049])
def test_small_and_ragged_sizes(builder, n):
    rec = trace.generate(trace.config("c1", 4096), interleave_solo=True)[:n]
    keys, pairs = builder.build(rec, time_ordered=True)
    okeys, opairs = O.build_pair_table(rec)
    assert_tables_match(keys, pairs, okeys, opairs)


def test_brute_force_agreement_with_ties_and_zero_durations(builder):
    rng = np.random.default_rng(5)
    n = 700
    start = np.sort(rng.integers(1000, 1400, n)).astype(np.uint64)  # many equal start_ns
    dur = rng.integers(0, 40, n).astype(np.uint64)  # including zero-length launches
    tenant = rng.integers(0, 3, n)
    solo = rng.random(n) < 0.3
    name = rng.integers(0, 6, n)
    rec = pack_records(name, np.ones((n, 3)), np.ones((n, 3)) * 32, np.zeros(n), tenant, solo, start, start + dur)
    keys, pairs = builder.build(rec)
    okeys, opairs = O.build_pair_table_bruteforce(rec)
    bkeys, bpairs = O.build_pair_table(rec)
    assert_tables_match(keys, pairs, bkeys, bpairs)
    for c in ("key_a", "key_b", "count", "median_a", "median_b", "min_a", "max_b", "efficiency"):
        assert np.array_equal(pairs[c], opairs[c], equal_nan=True), c


def test_hot_pair_large_segments(builder):
    # two keys only: every pair lands in one row, so the CTA-per-row selection path carries the medians
    rng = np.random.default_rng(9)
    n = 120_000
    tenant = (np.arange(n) % 2)
    dur = rng.integers(500, 5000, n).astype(np.uint64)
    start = (np.cumsum(rng.integers(100, 1500, n))).astype(np.uint64)
    solo = np.zeros(n, bool)
    solo[:2000] = True
    rec = pack_records(tenant, np.ones((n, 3)), np.ones((n, 3)) * 64, np.zeros(n), tenant, solo, start, start + dur)
    keys, pairs = builder.build(rec)
    okeys, opairs = O.build_pair_table(rec)
    assert len(opairs["count"]) == 1 and opairs["count"][0] > 50_000
    assert_tables_match(keys, pairs, okeys, opairs)


def test_error_statuses(builder):
    from kernel_scheduling_b200 import _lib

    rec = trace.generate(trace.config("c1", 5000))
    bad = rec.copy()
    bad["end_ns"][17] = bad["start_ns"][17] - 1
    with pytest.raises(_lib.KsError) as e:
        builder.build(bad)
    assert e.value.status == _lib.ERR_RECORD
    long = rec.copy()
    long["end_ns"][5] = long["start_ns"][5] + (1 << 31)
    with pytest.raises(_lib.KsError) as e:
        builder.build(long)
    assert e.value.status == _lib.ERR_RECORD
    with pytest.raises(_lib.KsError) as e:
        builder.build(trace.shuffled(rec), time_ordered=True)
    assert e.value.status == _lib.ERR_NOT_ORDERED
    # the handle stays usable after an error
    keys, pairs = builder.build(rec, time_ordered=True)
    okeys, opairs = O.build_pair_table(rec)
    assert_tables_match(keys, pairs, okeys, opairs)


def test_sparse_trace_uses_64_bit_windows(builder):
    # bursts of launches separated by idle gaps of 5 s: a join window then spans more than 2^31 ns
    rec = trace.generate(trace.config("c3", 40_000), interleave_solo=True)
    gap = (np.arange(len(rec), dtype=np.uint64) // np.uint64(64)) * np.uint64(5_000_000_000)
    rec["start_ns"] += gap
    rec["end_ns"] += gap
    keys, pairs = builder.build(rec, time_ordered=True)
    okeys, opairs = O.build_pair_table(rec)
    assert opairs["count"].sum() > 10_000
    assert_tables_match(keys, pairs, okeys, opairs)


def test_shape_changes_between_calls(builder):
    # with time-ordered input a call sizes its launches from what the previous call saw and verifies the guess at the
    # end; a trace that is larger, has more keys or fewer rows than the last one must give the same table as ever
    for cfg, n in (("c1", 20_000), ("c2", 300_000), ("c1", 5_000), ("c3", 150_000), ("c3", 150_000)):
        rec = trace.generate(trace.config(cfg, n))
        keys, pairs = builder.build(rec, time_ordered=True)
        okeys, opairs = O.build_pair_table(rec)
        assert_tables_match(keys, pairs, okeys, opairs)


def test_row_capacity_is_an_error_not_a_fault():
    from kernel_scheduling_b200 import _lib
    from kernel_scheduling_b200.pair_table import PairTableBuilder

    rec = trace.generate(trace.config("c1", 20_000))
    with PairTableBuilder(device=0, max_pair_rows=16) as small:
        for _ in range(2):  # the second call takes the path that trusts the previous call's counts
            with pytest.raises(_lib.KsError) as e:
                small.build(rec, time_ordered=True)
            assert e.value.status in (_lib.ERR_TOO_LARGE, _lib.ERR_TABLE_FULL)
        tiny = rec[:40]
        keys, pairs = small.build(tiny, time_ordered=True)
        okeys, opairs = O.build_pair_table(tiny)
        assert_tables_match(keys, pairs, okeys, opairs)


def test_pinned_buffers(builder):
    rec = trace.generate(trace.config("c1", 30_000))
    buf = builder.pinned_records(len(rec))
    buf[:] = rec
    keys, pairs = builder.build(buf, time_ordered=True, pinned=True)
    okeys, opairs = O.build_pair_table(rec)
    assert_tables_match(keys, pairs, okeys, opairs)


@pytest.mark.parametrize("cfg,n,min_pairs", [("c2", 10_000_000, 4_000_000), ("c3", 12_000_000, 20_000_000)])
def test_benchmark_sizes_match_oracle(builder, cfg, n, min_pairs):
    """The benchmark shapes at sizes where every sort pass, every row class (rows of millions of samples beside millions of
    rows of one) and the call that trusts the previous call's counts are at work together, against the C oracle."""
    rec = trace.generate_fast(trace.config(cfg, n))
    okeys, opairs = CO.build_pair_table(rec)
    assert int(opairs["count"].sum()) >= min_pairs and int(opairs["count"].max()) > 8192
    for call in range(2):  # the second call queues every stage from the first call's counts
        keys, pairs = builder.build(rec, time_ordered=True)
        assert_tables_match(keys, pairs, okeys, opairs)
        assert builder.info["n_pairs"] == int(opairs["count"].sum())
    # another trace of the same shape right behind it: the counts guessed from the last call are close but not equal
    rec2 = trace.generate_fast(trace.config(cfg, n // 2), window=1)
    keys, pairs = builder.build(rec2, time_ordered=True)
    assert_tables_match(keys, pairs, *CO.build_pair_table(rec2))


def test_full_size_c2_properties(builder):
    """The 10 M-record configuration: properties that hold whatever the oracle says."""
    rec = trace.generate_fast(trace.config("c2"))
    keys, pairs = builder.build(rec, time_ordered=True)
    info = dict(builder.info)
    assert info["n_records"] == len(rec) == 10_000_000
    assert int(keys["launches"].sum()) == len(rec)                       # every launch is counted under exactly one key
    assert int(keys["solo_launches"].sum()) == info["n_solo"]
    assert int(pairs["count"].sum()) == info["n_pairs"]                   # every overlapping pair lands in exactly one row
    assert (np.diff(keys["key"].astype(np.uint64).view(np.int64)) != 0).all() and (keys["key"][1:] > keys["key"][:-1]).all()
    order = np.lexsort((pairs["key_b"], pairs["key_a"]))
    assert (order == np.arange(len(pairs))).all()                         # rows sorted by (key_a, key_b), no duplicates
    assert len(np.unique(np.stack([pairs["key_a"], pairs["key_b"]], axis=1), axis=0)) == len(pairs)
    tenant_of = dict(zip(keys["key"].tolist(), keys["tenant"].tolist()))
    assert all(tenant_of[a] < tenant_of[b] for a, b in zip(pairs["key_a"][:2000].tolist(), pairs["key_b"][:2000].tolist()))
    for side in "ab":
        ok = (pairs["flags"] >> (0 if side == "a" else 1)) & 1 == 1
        mn, md, mx, mean = (pairs[f"{c}_{side}"][ok] for c in ("min", "median", "max", "mean"))
        assert (mn <= md).all() and (md <= mx).all() and (mn <= mean * (1 + 1e-12)).all() and (mean <= mx * (1 + 1e-12)).all()
        assert np.isnan(pairs[f"median_{side}"][~ok]).all()
        single = ok & (pairs["count"] == 1)
        assert np.array_equal(pairs[f"min_{side}"][single], pairs[f"max_{side}"][single])
        assert np.array_equal(pairs[f"median_{side}"][single], pairs[f"min_{side}"][single])
    # the same launches in another order give the same table bit for bit (exact columns) -- the sort in front is exercised
    keys2, pairs2 = builder.build(trace.shuffled(rec), time_ordered=False)
    assert keys2.tobytes() == keys.tobytes()
    for c in pairs.dtype.names:
        if c.startswith(("sum", "mean")):
            assert np.allclose(pairs2[c], pairs[c], rtol=1e-6, atol=0, equal_nan=True), c
        else:
            assert np.array_equal(pairs2[c], pairs[c], equal_nan=True), c


def _streamed(builder, rec, **kw):
    import torch

    dev = torch.from_numpy(rec.view(np.uint8).reshape(-1).copy()).cuda() if len(rec) else None
    builder.build_streamed_device(dev.data_ptr() if len(rec) else 0, len(rec), **kw) if len(rec) else builder.build_streamed_device(rec, **kw)
    return builder.fetch()


@pytest.mark.parametrize("cfg,n,window,parts", [("c1", 60_000, 7_000, 3), ("c2", 400_000, 150_000, 16), ("c3", 300_000, 40_000, 5), ("c4", 2_000_000, 300_000, 7)])
def test_streamed_build_equals_oracle(builder, cfg, n, window, parts):
    """Windows much smaller than the trace, launches that overlap across window ends, key ranges reduced one by one."""
    rec = trace.generate_fast(trace.config(cfg, n))
    keys, pairs = _streamed(builder, rec, window_records=window, n_parts=parts)
    okeys, opairs = CO.build_pair_table(rec)
    assert_tables_match(keys, pairs, okeys, opairs)
    assert builder.info["n_pairs"] == int(opairs["count"].sum()) and builder.info["n_rows"] == len(pairs)
    # ... and the ordinary call on the same handle afterwards
    keys1, pairs1 = builder.build(rec, time_ordered=True)
    assert keys1.tobytes() == keys.tobytes()
    assert_tables_match(keys1, pairs1, okeys, opairs)


def test_streamed_build_edge_cases(builder):
    from kernel_scheduling_b200 import _lib

    rec = trace.generate(trace.config("c1", 5000), interleave_solo=True)
    for m, window, parts in ((0, 100, 4), (1, 100, 4), (2, 1, 2), (777, 50, 16), (5000, 5000, 1), (5000, 100_000, 0)):
        keys, pairs = _streamed(builder, rec[:m], window_records=window, n_parts=parts)
        assert_tables_match(keys, pairs, *O.build_pair_table(rec[:m]))
    keys, pairs = _streamed(builder, rec, window_records=600, n_parts=3, key_type=True)
    assert_tables_match(keys, pairs, *O.build_pair_table(rec, key_mode=O.KEY_TYPE))
    # a launch that spans every window
    n = 4000
    start = np.arange(n, dtype=np.uint64) * 100 + 1000
    dur = np.full(n, 60, dtype=np.uint64)
    tenant = 1 + (np.arange(n) % 2)
    tenant[3], dur[3] = 0, 100 * n
    long = pack_records(tenant, np.ones((n, 3)), np.ones((n, 3)) * 32, np.zeros(n), tenant, np.zeros(n, bool), start, start + dur)
    keys, pairs = _streamed(builder, long, window_records=250, n_parts=4)
    assert_tables_match(keys, pairs, *O.build_pair_table(long))
    with pytest.raises(_lib.KsError) as e:
        _streamed(builder, trace.shuffled(rec), window_records=1000, n_parts=2)
    assert e.value.status == _lib.ERR_NOT_ORDERED
    keys, pairs = builder.build(rec, time_ordered=True)  # the handle stays usable
    assert_tables_match(keys, pairs, *O.build_pair_table(rec))


def test_committed_pair_tables(builder):
    """The CUDA path against the committed fixture of the main path (records in, table out), SHAPE and TYPE keys."""
    import os

    from tests.helpers import load_golden_pair_tables

    cases = load_golden_pair_tables(os.path.join(os.path.dirname(__file__), "golden", "pair_table_small.npz"))
    for tag, (rec, mode, gkeys, gpairs) in cases.items():
        keys, pairs = builder.build(rec, key_type=(mode == O.KEY_TYPE))
        assert_tables_match(keys, pairs, gkeys, gpairs)
        keys, pairs = builder.build(rec, key_type=(mode == O.KEY_TYPE), time_ordered=True)
        assert_tables_match(keys, pairs, gkeys, gpairs)
