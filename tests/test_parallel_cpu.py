"""CPU: the multi-rank orchestration (kernel_scheduling_b200.parallel) with a numpy stand-in for the per-rank kernels --
in one process for several world sizes, and as two gloo ranks."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

from kernel_scheduling_b200 import parallel, trace
from kernel_scheduling_b200.records import pack_records
from oracle import pair_table_oracle as O
from tests.fake_stages import FakeStages
from tests.helpers import assert_tables_match

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def sharded(rec, world, key_type=False):
    wins = parallel.split_windows(len(rec), world)
    gens = [parallel.build_steps(FakeStages(rec[lo:hi]), r, world, key_type) for r, (lo, hi) in enumerate(wins)]
    return parallel.run_in_process(gens)


def test_choose_splitters():
    hist = np.zeros(parallel.HIST_BINS, dtype=np.int64)
    hist[[3, 10, 11, 500]] = [100, 100, 100, 100]
    assert parallel.choose_splitters(hist, 1) == []
    sp = parallel.choose_splitters(hist, 4)
    dest = [sum(s <= b for s in sp) for b in (3, 10, 11, 500)]
    assert dest == [0, 1, 2, 3]
    hot = np.zeros(parallel.HIST_BINS, dtype=np.int64)
    hot[7] = 1000  # one bin holds everything: it is never split, some ranks get nothing
    sp = parallel.choose_splitters(hot, 4)
    assert sp == sorted(sp) and len({sum(s <= 7 for s in sp)}) == 1


def test_split_windows():
    assert parallel.split_windows(10, 3) == [(0, 4), (4, 7), (7, 10)]
    assert parallel.split_windows(2, 4) == [(0, 1), (1, 2), (2, 2), (2, 2)]


@pytest.mark.parametrize("world", [1, 2, 3, 4])
def test_sharded_table_equals_single_process_oracle(world):
    rec = trace.generate(trace.config("c3", 3000), interleave_solo=True)
    okeys, opairs = O.build_pair_table(rec)
    for keys, pairs in sharded(rec, world):
        assert_tables_match(keys, pairs, okeys, opairs)


def test_launch_spanning_several_windows():
    # tenant 0: one launch that runs across all four windows; tenants 1, 2: short launches everywhere
    n = 400
    start = np.arange(n, dtype=np.uint64) * 100 + 1000
    dur = np.full(n, 60, dtype=np.uint64)
    tenant = 1 + (np.arange(n) % 2)
    tenant[3], dur[3] = 0, 100 * n  # the long one
    solo = np.zeros(n, bool)
    rec = pack_records(tenant, np.ones((n, 3)), np.ones((n, 3)) * 32, np.zeros(n), tenant, solo, start, start + dur)
    okeys, opairs = O.build_pair_table(rec)
    assert opairs["count"].sum() > n - 10
    for keys, pairs in sharded(rec, 4):
        assert_tables_match(keys, pairs, okeys, opairs)


def test_type_keys_and_empty_windows():
    rec = trace.generate(trace.config("c1", 600))
    okeys, opairs = O.build_pair_table(rec, key_mode=O.KEY_TYPE)
    for keys, pairs in sharded(rec, 2, key_type=True):
        assert_tables_match(keys, pairs, okeys, opairs)
    tiny = rec[:3]
    okeys, opairs = O.build_pair_table(tiny)
    for keys, pairs in sharded(tiny, 4):  # windows 3 is empty
        assert_tables_match(keys, pairs, okeys, opairs)


def test_two_gloo_ranks(tmp_path):
    port = socket.socket()
    port.bind(("127.0.0.1", 0))
    p = port.getsockname()[1]
    port.close()
    script = os.path.join(ROOT, "tests", "gloo_rank.py")
    procs = [subprocess.Popen([sys.executable, script, str(r), "2", str(p), str(tmp_path)], cwd=ROOT) for r in range(2)]
    assert [q.wait(timeout=240) for q in procs] == [0, 0]
    rec = trace.generate(trace.config("c3", 2500))
    okeys, opairs = O.build_pair_table(rec)
    for r in range(2):
        d = np.load(tmp_path / f"rank{r}.npz")
        assert_tables_match(d["keys"], d["pairs"], okeys, opairs)
