"""GPU: the resident table (ks_update_*): after every window the table read out equals the oracle's table over all launches
so far -- bit for bit where the batch path is (counts, keys, min, max, medians), 1e-6 on sums and means."""
import numpy as np
import pytest

from kernel_scheduling_b200 import _lib, trace
from kernel_scheduling_b200.pair_table import PairTableBuilder
from kernel_scheduling_b200.records import pack_records
from oracle import pair_table_oracle as O
from tests.helpers import assert_tables_match

pytestmark = pytest.mark.gpu


def _feed(b, rec, cuts, check_every=1, key_mode=O.KEY_SHAPE):
    lo = 0
    for i, hi in enumerate(cuts):
        b.update(rec[lo:hi])
        lo = hi
        if (i + 1) % check_every == 0 or hi == cuts[-1]:
            keys, pairs = b.update_table()
            okeys, opairs = O.build_pair_table(rec[:hi], key_mode=key_mode)
            assert_tables_match(keys, pairs, okeys, opairs)


@pytest.mark.parametrize("cfg,n,windows", [("c5", 40_000, 10), ("c1", 30_000, 7), ("c3", 24_000, 12)])
def test_resident_table_equals_batch_table_after_every_window(cfg, n, windows):
    spec = trace.config(cfg, n)
    if cfg == "c3":
        for t in spec.tenants:
            t.n_keys = 400  # a session holds 2,048 keys
    rec = trace.generate(spec, interleave_solo=True)  # solo launches throughout, as in a live profiling run
    cuts = [int(x) for x in np.linspace(0, n, windows + 1)[1:]]
    with PairTableBuilder(device=0) as b:
        b.update_begin()
        _feed(b, rec, cuts)
        assert b.update_info["ms_total"] > 0
        b.update_end()


def test_resident_table_hot_rows_many_windows_and_type_keys():
    # two keys per tenant: every row gets thousands of samples, far more than the 64 values a row keeps, over 40 windows of
    # uneven size (1 .. 3,000 launches); TYPE keys
    rng = np.random.default_rng(3)
    n = 36_000
    tenant = rng.integers(0, 3, n)
    gap = rng.integers(50, 400, n)
    start = np.cumsum(gap).astype(np.uint64) + np.uint64(10_000)
    dur = (rng.lognormal(6.0, 0.5, n)).astype(np.uint64) + np.uint64(20)
    names = tenant * 2 + rng.integers(0, 2, n)
    solo = rng.random(n) < 0.15
    rec = pack_records(names, rng.integers(1, 5, (n, 3)), np.full((n, 3), 64), np.zeros(n), tenant, solo, start, start + dur)
    cuts = sorted(set(int(x) for x in np.concatenate([[1, 2, 5, 70], rng.integers(100, n, 34), [n]])))
    with PairTableBuilder(device=0) as b:
        b.update_begin(key_type=True)
        _feed(b, rec, cuts, check_every=6, key_mode=O.KEY_TYPE)
        b.update_end()


def test_launch_spanning_many_windows_is_carried():
    n = 6000
    start = np.arange(n, dtype=np.uint64) * 100 + 1000
    dur = np.full(n, 60, dtype=np.uint64)
    tenant = 1 + (np.arange(n) % 2)
    tenant[3], dur[3] = 0, 100 * n  # runs through every later window
    tenant[2500], dur[2500] = 0, 100 * 700
    rec = pack_records(tenant, np.ones((n, 3)), np.ones((n, 3)) * 32, np.zeros(n), tenant, np.zeros(n, bool), start, start + dur)
    with PairTableBuilder(device=0) as b:
        b.update_begin()
        _feed(b, rec, list(range(500, n + 1, 500)), check_every=4)
        b.update_end()


def test_session_errors():
    rec = trace.generate(trace.config("c1", 4000))
    with PairTableBuilder(device=0) as b:
        with pytest.raises(_lib.KsError) as e:
            b.update(rec[:100])  # no session
        assert e.value.status == _lib.ERR_ARG
        b.update_begin()
        b.update(rec[:2000])
        with pytest.raises(_lib.KsError) as e:
            b.update(rec[1000:3000])  # starts before the end of the previous window
        assert e.value.status == _lib.ERR_NOT_ORDERED
        with pytest.raises(_lib.KsError) as e:
            b.update_table()  # the session is over after an error
        assert e.value.status == _lib.ERR_REBUILD
        b.update_begin()  # and a new one works
        b.update(rec)
        assert_tables_match(*b.update_table(), *O.build_pair_table(rec))
        b.update_end()


def test_a_jump_of_a_rows_distribution_is_reported_not_hidden():
    # 40,000 solo launches of one kernel around 1,000 ns (the row keeps the central 16,384 values), then 40,000 in ONE window
    # around 50,000 ns: the median moves to a value the row no longer keeps.  The library must say so.
    n1, n2 = 40_000, 40_000
    dur = np.concatenate([np.full(n1, 1000) + np.arange(n1) % 7, np.full(n2, 50_000) + np.arange(n2) % 11]).astype(np.uint64)
    n = n1 + n2
    start = np.arange(n, dtype=np.uint64) * 100_000 + 1000
    rec = pack_records(np.zeros(n), np.ones((n, 3)), np.ones((n, 3)) * 32, np.zeros(n), np.zeros(n), np.ones(n, bool), start, start + dur)
    with PairTableBuilder(device=0) as b:
        b.update_begin()
        for lo in range(0, n1, 8000):
            b.update(rec[lo: lo + 8000])
        keys, _ = b.update_table()
        assert keys["solo_ns"][0] == O.build_pair_table(rec[:n1])[0]["solo_ns"][0]
        with pytest.raises(_lib.KsError) as e:
            b.update(rec[n1:])
        assert e.value.status == _lib.ERR_REBUILD
        b.update_end()


def test_online_driver_verifies_publishes_and_takes_host_windows():
    """The online configuration's driver at a small size: stretches generated beside the GPU, the table at the end equal to
    a batch build over every launch (verify), the last windows arriving in pinned host memory, and the table republished in
    the shared-memory segment every few windows."""
    import os

    from kernel_scheduling_b200 import online, pair_table_shm

    name = f"/ks_test_online_{os.getpid()}"
    try:
        res = online.run(windows=24, per=4096, verify=True, publish_every=8, host_windows=4, shm_name=name)
        assert res["verified_against_batch_build"] is True
        assert res["records"] == 24 * 4096 and res["windows"] == 24
        assert res["host_windows"]["windows"] == 4 and res["publish"]["times"] == 3
        assert res["p50"] > 0 and res["device_ms_p50"] > 0 and res["pair_rows"] > 0
        with pair_table_shm.Attached(name) as seg:
            assert seg.generation == 24  # the last publication: after window 24
    finally:
        pair_table_shm.unlink(name)


def test_online_stretches_are_ordered_and_reproducible():
    from kernel_scheduling_b200 import online

    got = list(online.stretches(7, 512))
    old = online.STRETCH_WINDOWS
    try:
        online.STRETCH_WINDOWS = 3  # three stretches of 3, 3 and 1 windows
        parts = list(online.stretches(7, 512))
    finally:
        online.STRETCH_WINDOWS = old
    assert [f for f, _ in got] == [0] and [f for f, _ in parts] == [0, 3, 6]
    assert sum(len(r) for _, r in parts) == 7 * 512 == len(got[0][1])
    allrec = np.concatenate([r for _, r in parts])
    assert np.all(np.diff(allrec["start_ns"].astype(np.int64)) >= 0)  # stretches follow one another in time
    again = np.concatenate([r for _, r in online.stretches(7, 512)])
    assert again.tobytes() == got[0][1].tobytes()
