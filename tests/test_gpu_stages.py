"""Each kernel family through its own C-ABI entry point against numpy on the same seeded inputs."""
import numpy as np
import pytest

from kernel_scheduling_b200 import trace
from oracle import pair_table_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [0, 1, 255, 256, 257, 100_003])
@pytest.mark.parametrize("key_type", [False, True])
def test_hash_keys(builder, n, key_type):
    rec = trace.generate(trace.config("c3", max(n, 4096)))[:n]
    got = builder.hash_keys(rec, key_type=key_type)
    assert np.array_equal(got, O.kernel_keys(rec, O.KEY_TYPE if key_type else O.KEY_SHAPE))


@pytest.mark.parametrize("dtype", [np.uint32, np.uint64])
@pytest.mark.parametrize("n", [0, 1, 2, 4095, 4096, 4097, 250_001])
def test_sort_pairs_full_width(builder, dtype, n):
    rng = np.random.default_rng(n + 1)
    keys = rng.integers(0, np.iinfo(dtype).max, n, dtype=dtype, endpoint=True)
    vals = np.arange(n, dtype=dtype)
    k, v = builder.sort_pairs(keys, vals)
    order = np.argsort(keys, kind="stable")
    assert np.array_equal(k, keys[order])
    assert np.array_equal(v, vals[order])  # stability: equal keys keep their input order


@pytest.mark.parametrize("bits", [(0, 3), (0, 11), (5, 22), (8, 16)])
def test_sort_pairs_bit_ranges_and_skew(builder, bits):
    rng = np.random.default_rng(3)
    n = 300_000
    keys = (rng.zipf(1.3, n) % (1 << 24)).astype(np.uint32)  # heavy duplicates
    vals = np.arange(n, dtype=np.uint32)
    k, v = builder.sort_pairs(keys, vals, bits[0], bits[1])
    field = (keys >> bits[0]) & ((1 << (bits[1] - bits[0])) - 1)
    order = np.argsort(field, kind="stable")
    assert np.array_equal(k, keys[order])
    assert np.array_equal(v, vals[order])


def test_sort_keys_only(builder):
    rng = np.random.default_rng(4)
    keys = rng.integers(0, 1 << 40, 70_000, dtype=np.uint64)
    k, v = builder.sort_pairs(keys, None, 0, 40)
    assert v is None and np.array_equal(k, np.sort(keys))


@pytest.mark.parametrize("shuffle", [False, True])
def test_sort_launches(builder, shuffle):
    rec = trace.generate(trace.config("c1", 80_000))
    if shuffle:
        rec = trace.shuffled(rec)
    keys, start = builder.sort_launches(rec)
    okeys = O.kernel_keys(rec)
    order = np.lexsort((rec["start_ns"], okeys))
    assert np.array_equal(keys, okeys[order])
    assert np.array_equal(start, rec["start_ns"][order])


@pytest.mark.parametrize("cfg,n", [("c1", 30_000), ("c3", 50_000), ("c4", 40_000)])
def test_join_overlaps(builder, cfg, n):
    rec = trace.generate(trace.config(cfg, n), interleave_solo=(cfg == "c3"))
    ia, ib = builder.join_overlaps(rec)
    # independent restatement: all pairs by per-tenant searchsorted, then compared as sets of (a, b) positions
    order = np.argsort(rec["start_ns"], kind="stable")
    r = rec[order]
    solo = (r["smem_word"] & (1 << 23)) != 0
    ten = r["smem_word"] >> 24
    s, e = r["start_ns"], r["end_ns"]
    want = set()
    idx = np.flatnonzero(~solo)
    hi = np.searchsorted(s, e[idx], side="left")
    for i, h in zip(idx, hi):
        for j in range(i + 1, h):
            if not solo[j] and ten[j] != ten[i] and s[i] < e[j]:
                want.add((i, j) if ten[i] < ten[j] else (j, i))
    got = set(zip(ia.tolist(), ib.tolist()))
    assert len(got) == len(ia), "a pair was emitted twice"
    assert got == want


def test_segment_stats(builder):
    rng = np.random.default_rng(11)
    sizes = np.concatenate([rng.integers(0, 40, 3000), [0, 1, 2, 32, 33, 1000, 4097, 50_000, 0]])
    offsets = np.concatenate([[0], np.cumsum(sizes)]).astype(np.uint64)
    values = rng.integers(0, 1 << 31, int(offsets[-1]), dtype=np.uint32)
    # a segment of equal values, one with a narrow range (few differing bits), one spanning the full range
    values[offsets[-4]: offsets[-4] + 4097] = 77
    values[offsets[-3]: offsets[-3] + 50_000] = rng.integers(1_000_000, 1_000_900, 50_000)
    got = builder.segment_stats(values, offsets)
    for sidx in range(len(sizes)):
        seg = np.sort(values[int(offsets[sidx]): int(offsets[sidx + 1])].astype(np.uint64))
        c = len(seg)
        want = [c, seg.sum(), seg[0], seg[-1], seg[(c - 1) // 2], seg[c // 2]] if c else [0, 0, 0, 0, 0, 0]
        assert got[sidx].tolist() == [int(x) for x in want], (sidx, c)


def test_count_batches(builder):
    rng = np.random.default_rng(2)
    s1 = rng.choice(np.arange(1, 400_000, dtype=np.uint64) * 7 + (1 << 41), 90_000, replace=False)
    s2 = np.concatenate([rng.choice(s1, 20_000, replace=False), rng.choice(np.arange(1, 400_000, dtype=np.uint64) * 7 + 3 + (1 << 41), 50_000, replace=False)])
    rng.shuffle(s2)
    assert builder.count_batches(s1, s2) == O.count_batches(s1, s2) == [90_000 - 20_000 + 50_000, 20_000]
    assert builder.count_batches(s1[:0], s2[:5]) == [5, 0]
    from kernel_scheduling_b200 import _lib

    with pytest.raises(_lib.KsError) as e:
        builder.count_batches(np.concatenate([s1, s1[:1]]), s2)
    assert e.value.status == _lib.ERR_DUPLICATE


def test_combine_duplicates(builder):
    rng = np.random.default_rng(8)
    rows, cols, groups = 5000, 9, 137
    g = rng.integers(0, groups, rows).astype(np.uint32)
    g[:groups] = np.arange(groups)
    w = rng.integers(1, 50, rows).astype(np.float64)
    v = rng.normal(10, 3, (rows, cols))
    v[rng.random((rows, cols)) < 0.2] = np.nan
    v[g == 5, 2] = np.nan  # an all-NaN group/column -> NaN
    total, means = builder.combine_duplicates(g, w, v, groups)
    _, _, ototal, omeans = O.combine_duplicates(g.tolist(), [0] * rows, w, v)
    assert np.array_equal(total, ototal)
    assert np.allclose(means, omeans, rtol=1e-12, atol=0, equal_nan=True)
    assert np.isnan(means[5, 2])


def test_unaligned_device_records_are_refused_before_any_launch(builder):
    """K1's bulk copies need a 16-byte-aligned source; a device pointer that is not (a slice of a byte buffer) must come
    back as KS_ERR_ARG from every entry point that decodes records -- no kernel is launched with it."""
    import ctypes

    import torch

    from kernel_scheduling_b200 import _lib

    lib = _lib.load()
    rec = trace.generate(trace.config("c1", 2000))
    buf = torch.zeros(len(rec) * 48 + 64, dtype=torch.uint8, device="cuda")
    buf[8: 8 + len(rec) * 48] = torch.from_numpy(rec.view(np.uint8).reshape(-1)).cuda()
    bad = ctypes.c_void_p(buf.data_ptr() + 8)
    out = torch.zeros(len(rec) * 2, dtype=torch.int64, device="cuda")
    o = ctypes.c_void_p(out.data_ptr())
    h, n, dev = builder._h, len(rec), _lib.ON_DEVICE
    calls = {
        "ks_build_table": lambda: lib.ks_build_table(h, bad, n, dev, None),
        "ks_hash_keys": lambda: lib.ks_hash_keys(h, bad, n, dev, o),
        "ks_sort_launches": lambda: lib.ks_sort_launches(h, bad, n, dev, o, o),
        "ks_join_overlaps": lambda: lib.ks_join_overlaps(h, bad, n, dev, None, None, 0),
        "ks_mg_begin": lambda: lib.ks_mg_begin(h, bad, n, 0),
    }
    for name, call in calls.items():
        assert call() == -_lib.ERR_ARG, name
        assert b"aligned" in lib.ks_last_error(h), name
    # the handle is as usable as before
    keys, pairs = builder.build(rec, time_ordered=True)
    assert len(keys) > 0


def test_a_wait_that_cannot_be_satisfied_runs_out_and_is_reported(builder):
    """The sort's look-back waits for earlier tiles with a bounded number of polls.  A pass whose first tile is never
    started must end by itself and come back as KS_ERR_WAIT; the handle works as before afterwards."""
    from kernel_scheduling_b200 import _lib

    lib = _lib.load()
    assert lib.ks_selftest_bounded_wait(builder._h) == -_lib.ERR_WAIT
    assert b"wait" in lib.ks_last_error(builder._h)
    rec = trace.generate(trace.config("c1", 3000))
    keys, pairs = builder.build(rec, time_ordered=True)
    okeys, opairs = O.build_pair_table(rec)
    assert np.array_equal(keys["key"], okeys["key"]) and np.array_equal(pairs["count"], opairs["count"])
