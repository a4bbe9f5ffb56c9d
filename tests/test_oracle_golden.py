"""CPU: the oracle against the reference's own outputs (golden vectors) and against independent restatements."""
import io
import json
import os

import numpy as np
import pandas as pd
import pytest

from kernel_scheduling_b200 import trace
from kernel_scheduling_b200.records import RECORD_DTYPE, pack_records
from oracle import pair_table_oracle as O

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_record_layout_is_shared():
    assert O.RECORD_DTYPE == RECORD_DTYPE and RECORD_DTYPE.itemsize == 48
    assert [RECORD_DTYPE.fields[f][1] for f in ("name_id", "grid", "block", "smem_word", "start_ns", "end_ns")] == [0, 4, 16, 28, 32, 40]


def test_mix64_known_answers():
    # splitmix64 from seed 0 (published test vector): outputs mix64(1 * G), mix64(2 * G), mix64(3 * G)
    g = 0x9E3779B97F4A7C15
    got = O.mix64(np.array([g, (2 * g) % 2**64, (3 * g) % 2**64], dtype=np.uint64))
    assert [int(x) for x in got] == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F]


def test_kernel_key_fields():
    rec = pack_records([7, 7, 7, 7, 8], [[1, 2, 3]] * 3 + [[9, 2, 3]] + [[1, 2, 3]], [[128, 1, 1]] * 5, [0, 0, 4096, 0, 0], [0, 1, 0, 0, 0],
                       [False, True, False, False, False], np.arange(5) * 10 + 100, np.arange(5) * 10 + 105)
    k = O.kernel_keys(rec)
    assert len(set(k.tolist())) == 5  # tenant, smem, grid and name all enter the SHAPE key
    rec2 = rec.copy()
    rec2["smem_word"] ^= np.uint32(1 << 23)  # the solo flag does not
    assert np.array_equal(O.kernel_keys(rec2), k)
    kt = O.kernel_keys(rec, O.KEY_TYPE)
    assert kt[0] == kt[2] == kt[3] and kt[0] != kt[1] and kt[0] != kt[4]  # TYPE: tenant + name + block only


@pytest.mark.parametrize("interleave", [False, True])
def test_vectorised_oracle_equals_brute_force(interleave):
    rec = trace.generate(trace.config("c3", 1200), interleave_solo=interleave)
    k1, p1 = O.build_pair_table(rec)
    k2, p2 = O.build_pair_table_bruteforce(rec)
    for c in ("key", "launches", "solo_launches", "solo_ns", "tenant"):
        assert np.array_equal(k1[c], k2[c], equal_nan=True), c
    assert len(p1["count"]) > 50
    for c in p2:
        if c.startswith(("sum", "mean")):
            assert np.allclose(p1[c], p2[c], rtol=1e-12, atol=0, equal_nan=True), c
        else:
            assert np.array_equal(p1[c], p2[c], equal_nan=True), c


def test_oracle_order_independent_and_rejects_bad_records():
    rec = trace.generate(trace.config("c1", 3000))
    _, p1 = O.build_pair_table(rec)
    _, p2 = O.build_pair_table(trace.shuffled(rec))
    for c in p1:
        assert np.allclose(p1[c], p2[c], rtol=1e-12, atol=0, equal_nan=True) if p1[c].dtype.kind == "f" else np.array_equal(p1[c], p2[c]), c
    bad = rec.copy()
    bad["end_ns"][3] = bad["start_ns"][3] - 1
    with pytest.raises(ValueError):
        O.build_pair_table(bad)


def test_count_batches_matches_reference_stdout():
    cases = json.load(open(os.path.join(GOLDEN, "postprocess_cases.json")))
    assert len(cases) >= 6
    for c in cases:
        s1, s2 = np.array(c["start1"], dtype=np.uint64), np.array(c["start2"], dtype=np.uint64)
        if c["assertion"]:
            with pytest.raises(ValueError):
                O.count_batches(s1, s2)
        else:
            assert str(O.count_batches(s1, s2)) == c["stdout"].strip().splitlines()[-1], c["name"]


@pytest.mark.parametrize("case", [0, 1])
def test_combine_duplicates_matches_reference_csv(case):
    df = pd.read_csv(os.path.join(GOLDEN, f"combine_in_{case}.csv"))
    want = pd.read_csv(os.path.join(GOLDEN, f"combine_out_{case}.csv"))
    excl = ["Launches", "Grid", "Shared Mem Pipe %", "Shared Mem Pipe % std", "Kernel", "Block"]
    cols = [c for c in df.columns if c not in excl]
    gk, gb, total, means = O.combine_duplicates(df["Kernel"].tolist(), df["Block"].tolist(), df["Launches"].to_numpy(), df[cols].to_numpy(dtype=np.float64))
    assert gk == want["Kernel"].tolist() and gb == want["Block"].tolist()
    assert np.array_equal(total, want["Launches"].to_numpy())
    assert list(want.columns) == ["Kernel", "Block", "Launches"] + cols
    assert np.allclose(means, want[cols].to_numpy(), rtol=1e-12, atol=0, equal_nan=True)


def test_trace_generator_shapes():
    spec = trace.config("c2", 200_000)
    rec = trace.generate(spec)
    assert len(rec) == 200_000 and (np.diff(rec["start_ns"].astype(np.int64)) >= 0).all()
    solo = (rec["smem_word"] & (1 << 23)) != 0
    assert abs(solo.mean() - 0.10) < 0.01
    ten = rec["smem_word"] >> 24
    for t in (0, 1):  # one launch in flight per tenant: its co-run intervals never overlap each other
        m = (ten == t) & ~solo
        assert (rec["start_ns"][m][1:] >= rec["end_ns"][m][:-1]).all()
    k, p = O.build_pair_table(rec, check_bijection=False)
    assert len(k["key"]) <= 2000 and 0.3 < p["count"].sum() / len(rec) < 0.7


def _ncu_pool_inputs():
    """Per-launch values of real Nsight Compute reports (extracted with the reference script's helpers) -> the label
    frame the pooling takes, and the summary CSV the reference script wrote for the same reports."""
    import pandas as pd

    from kernel_scheduling_b200 import ncu_summary as N

    launches = pd.read_csv(os.path.join(GOLDEN, "ncu_launches.csv"), float_precision="round_trip")
    ref = pd.read_csv(os.path.join(GOLDEN, "ncu_summary_ref.csv"), float_precision="round_trip")  # the default parser is off by an ulp now and then
    bpw, ratio = N.per_launch_labels(launches["duration_us"], launches["waves"], launches["grid_total"])
    frame = launches[["Kernel", "Block"]].copy()
    frame[N.RATIO_LABEL] = ratio
    frame[N.BPW_LABEL] = bpw
    for c in launches.columns[5:]:
        frame[c] = launches[c]
    return frame, ref


def test_pooling_oracle_equals_the_reference_script_on_real_reports():
    frame, ref = _ncu_pool_inputs()
    labels = [c for c in frame.columns if c not in ("Kernel", "Block")]
    assert [c for c in ref.columns[3:]] == [x for l in labels for x in (l, f"{l} std")]
    keys = list(zip(ref["Kernel"], ref["Block"]))  # the reference's group order
    gid = np.array([keys.index(kb) for kb in zip(frame["Kernel"], frame["Block"])])
    launches, mean, std = O.pool_launches(gid, frame[labels].to_numpy(dtype=np.float64), len(keys))
    assert list(launches) == list(ref["Launches"])
    for j, l in enumerate(labels):
        assert np.array_equal(mean[:, j], ref[l].to_numpy(dtype=np.float64), equal_nan=True), l
        assert np.array_equal(std[:, j], ref[f"{l} std"].to_numpy(dtype=np.float64), equal_nan=True), l


# ---- the C restatement (oracle/pair_table_oracle.c) is kept equal to the numpy oracle, column by column
def _assert_oracles_equal(rec, key_mode=0):
    from oracle import c_oracle as CO

    k1, p1 = O.build_pair_table(rec, key_mode=key_mode)
    k2, p2 = CO.build_pair_table(rec, key_mode=key_mode)
    assert set(k1) == set(k2) and set(p1) == set(p2)
    for c in k1:
        assert np.array_equal(k1[c], k2[c], equal_nan=True), c
    for c in p1:
        if c.startswith(("sum", "mean")):
            assert np.allclose(p1[c], p2[c], rtol=1e-12, atol=0, equal_nan=True), c
        else:
            assert np.array_equal(p1[c], p2[c], equal_nan=True), c
    return p1


@pytest.mark.parametrize("cfg,n", [("c1", 60_000), ("c2", 120_000), ("c3", 100_000), ("c4", 100_000)])
def test_c_oracle_equals_numpy_oracle(cfg, n):
    rec = trace.generate(trace.config(cfg, n))
    _assert_oracles_equal(rec)
    _assert_oracles_equal(trace.shuffled(rec), key_mode=O.KEY_TYPE)


def test_c_oracle_edge_cases():
    from oracle import c_oracle as CO

    spec = trace.config("c1", 30_000)
    spec.solo_fraction = 0.02  # keys without a baseline: NaN sides
    p = _assert_oracles_equal(trace.generate(spec, interleave_solo=True))
    assert (p["flags"] != 3).any() and (p["flags"] == 3).any()
    rng = np.random.default_rng(5)
    n = 700  # ties in start_ns, zero-length launches, three tenants
    start = np.sort(rng.integers(1000, 1400, n)).astype(np.uint64)
    dur = rng.integers(0, 40, n).astype(np.uint64)
    tenant = rng.integers(0, 3, n)
    rec = pack_records(rng.integers(0, 6, n), np.ones((n, 3)), np.ones((n, 3)) * 32, np.zeros(n), tenant, rng.random(n) < 0.3, start, start + dur)
    _assert_oracles_equal(rec)
    for m in (0, 1, 2, 33):
        _assert_oracles_equal(rec[:m])
    assert np.array_equal(CO.kernel_keys(rec), O.kernel_keys(rec)) and np.array_equal(CO.kernel_keys(rec, 1), O.kernel_keys(rec, 1))
    bad = rec.copy()
    bad["end_ns"][3] = bad["start_ns"][3] - 1
    with pytest.raises(ValueError):
        CO.build_pair_table(bad)
    bad = rec.copy()
    bad["end_ns"][3] = bad["start_ns"][3] + (1 << 31)
    with pytest.raises(ValueError):
        CO.build_pair_table(bad)


def test_fast_generator_is_ordered_deterministic_and_shaped_like_the_numpy_one():
    spec = trace.config("c3", 400_000)
    rec = trace.generate_fast(spec)
    assert len(rec) == 400_000 and rec.dtype == RECORD_DTYPE
    assert (np.diff(rec["start_ns"].astype(np.int64)) >= 0).all() and (rec["end_ns"] > rec["start_ns"]).all()
    assert rec.tobytes() == trace.generate_fast(spec, threads=3).tobytes() == trace.generate_fast(spec, threads=1).tobytes()
    assert rec.tobytes() != trace.generate_fast(spec, window=1).tobytes()
    ref = trace.generate(spec)
    # same key tables (a function of the seed), similar launch mix: keys, solo share, overlapping pairs per launch
    assert set(O.kernel_keys(rec).tolist()) <= set(O.kernel_keys(ref).tolist()) | set(O.kernel_keys(rec).tolist())
    solo = lambda r: float(((r["smem_word"] >> 23) & 1).mean())
    assert abs(solo(rec) - solo(ref)) < 0.01
    from oracle import c_oracle as CO

    pf = CO.build_pair_table(rec)[1]["count"].sum() / len(rec)
    pn = CO.build_pair_table(ref)[1]["count"].sum() / len(ref)
    assert abs(pf - pn) / pn < 0.05
    # within a tenant launches never overlap (one launch in flight per process)
    for t in range(4):
        m = (rec["smem_word"] >> 24) == t
        assert (rec["start_ns"][m][1:] >= rec["end_ns"][m][:-1]).all()


def test_oracles_equal_the_committed_pair_tables():
    """The main path's fixture (tests/golden/pair_table_small.npz: seeded traces and the tables the quadratic restatement
    gave when the fixture was made): the vectorised oracle and the C oracle still give exactly those tables."""
    from oracle import c_oracle as CO
    from tests.helpers import assert_columns_match, load_golden_pair_tables

    cases = load_golden_pair_tables(os.path.join(GOLDEN, "pair_table_small.npz"))
    assert set(cases) == {"c1", "c3", "c2type"}
    for tag, (rec, mode, gkeys, gpairs) in cases.items():
        assert rec.dtype == RECORD_DTYPE and len(gpairs["count"]) > 200
        keys, pairs = O.build_pair_table(rec, key_mode=mode)
        assert_columns_match(keys, pairs, gkeys, gpairs)
        ckeys, cpairs = CO.build_pair_table(rec, key_mode=mode)
        assert_columns_match(ckeys, cpairs, gkeys, gpairs)
