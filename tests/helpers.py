"""Shared comparison helpers for the parity tests."""
import numpy as np

EXACT_PAIR_COLS = ("key_a", "key_b", "count", "flags", "min_a", "max_a", "median_a", "min_b", "max_b", "median_b", "efficiency", "span_sum_ns")
CLOSE_PAIR_COLS = ("sum_a", "mean_a", "sum_b", "mean_b")
RTOL = 1e-6  # float sum and mean: the tolerance the path's contract states; everything else is bit-exact


def assert_tables_match(keys, pairs, okeys, opairs):
    """Library tables (structured arrays) against the oracle's columns."""
    assert len(keys) == len(okeys["key"])
    for c in ("key", "name_id", "grid", "block", "smem", "tenant", "launches", "solo_launches"):
        if c in okeys:
            assert np.array_equal(keys[c], okeys[c]), c
    assert np.array_equal(keys["solo_ns"], okeys["solo_ns"], equal_nan=True), "solo_ns"
    assert len(pairs) == len(opairs["count"]), (len(pairs), len(opairs["count"]))
    for c in EXACT_PAIR_COLS:
        assert np.array_equal(pairs[c], opairs[c], equal_nan=True), c
    for c in CLOSE_PAIR_COLS:
        assert np.allclose(pairs[c], opairs[c], rtol=RTOL, atol=0.0, equal_nan=True), c


def load_golden_pair_tables(path):
    """tests/golden/pair_table_small.npz -> {tag: (records, key_mode, key columns, pair columns)}."""
    z = np.load(path)
    cases = {}
    for name in z.files:
        tag, kind, *col = name.split(".")
        c = cases.setdefault(tag, {"keys": {}, "pairs": {}})
        if kind in ("keys", "pairs"):
            c[kind][col[0]] = z[name]
        else:
            c[kind] = z[name]
    return {tag: (c["records"], int(c["mode"]), c["keys"], c["pairs"]) for tag, c in cases.items()}


def assert_columns_match(keys, pairs, okeys, opairs):
    """Two oracle-style tables (dicts of columns) against each other, under the same contract as assert_tables_match."""
    assert set(okeys) <= set(keys) and set(opairs) <= set(pairs)  # (the quadratic restatement carries fewer key columns)
    for c in okeys:
        assert np.array_equal(keys[c], okeys[c], equal_nan=True), c
    for c in opairs:
        if c in CLOSE_PAIR_COLS:
            assert np.allclose(pairs[c], opairs[c], rtol=RTOL, atol=0.0, equal_nan=True), c
        else:
            assert np.array_equal(pairs[c], opairs[c], equal_nan=True), c
