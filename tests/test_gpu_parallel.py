"""GPU: the multi-rank path through the C ABI (ks_mg_*).  All ranks of a world run one after the other in this process
on one GPU (no kernel ever waits for another rank, so this is safe), collectives are fulfilled in-process; with two or
more GPUs present the same path also runs as real NCCL ranks."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch

from kernel_scheduling_b200 import parallel, trace
from kernel_scheduling_b200.pair_table import PairTableBuilder
from kernel_scheduling_b200.records import pack_records
from oracle import pair_table_oracle as O
from tests.helpers import assert_tables_match

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def sharded_gpu(rec, world, key_type=False):
    wins = parallel.split_windows(len(rec), world)
    stream = torch.cuda.Stream()  # the library and torch must share one stream (see parallel.GpuStages)
    with torch.cuda.stream(stream):
        builders = [PairTableBuilder(device=0, stream=stream.cuda_stream) for _ in range(world)]
        try:
            stages = [parallel.GpuStages(b, torch.from_numpy(rec[lo:hi].view(np.uint8).reshape(-1).copy()).cuda()) for b, (lo, hi) in zip(builders, wins)]
            return parallel.run_in_process([parallel.build_steps(s, r, world, key_type) for r, s in enumerate(stages)])
        finally:
            torch.cuda.synchronize()
            for b in builders:
                b.close()


@pytest.mark.parametrize("cfg,n,world", [("c1", 60_000, 1), ("c2", 300_000, 2), ("c3", 200_000, 4), ("c4", 150_000, 8)])
def test_sharded_table_equals_oracle(cfg, n, world):
    rec = trace.generate(trace.config(cfg, n))
    okeys, opairs = O.build_pair_table(rec)
    for keys, pairs in sharded_gpu(rec, world):
        assert_tables_match(keys, pairs, okeys, opairs)


def test_sharded_c4_shape_at_size_equals_oracle():
    """Eight time windows of a c4-shaped trace (8 tenants, 20,000 keys) large enough that every window carries a halo, the
    key ranges hold hundreds of thousands of rows each and the sample exchange moves millions of samples."""
    from oracle import c_oracle as CO

    rec = trace.generate_fast(trace.config("c4", 5_000_000))
    okeys, opairs = CO.build_pair_table(rec)
    assert len(okeys["key"]) == 20_000 and int(opairs["count"].sum()) > 15_000_000
    for keys, pairs in sharded_gpu(rec, 8)[:2]:  # every rank holds the whole table; two of them are compared in full
        assert_tables_match(keys, pairs, okeys, opairs)


def test_sharded_equals_single_gpu_bit_for_bit(builder):
    rec = trace.generate(trace.config("c3", 120_000), interleave_solo=True)
    keys1, pairs1 = builder.build(rec, time_ordered=True)
    for keys, pairs in sharded_gpu(rec, 3):
        assert keys.tobytes() == keys1.tobytes()
        for c in pairs1.dtype.names:
            if c.startswith(("sum", "mean")):
                assert np.allclose(pairs[c], pairs1[c], rtol=1e-6, atol=0, equal_nan=True)
            else:
                assert np.array_equal(pairs[c], pairs1[c], equal_nan=True), c


def test_launch_spanning_windows_and_type_keys():
    n = 4000
    start = np.arange(n, dtype=np.uint64) * 100 + 1000
    dur = np.full(n, 60, dtype=np.uint64)
    tenant = 1 + (np.arange(n) % 2)
    tenant[3], dur[3] = 0, 100 * n
    rec = pack_records(tenant, np.ones((n, 3)), np.ones((n, 3)) * 32, np.zeros(n), tenant, np.zeros(n, bool), start, start + dur)
    okeys, opairs = O.build_pair_table(rec, key_mode=O.KEY_TYPE)
    for keys, pairs in sharded_gpu(rec, 4, key_type=True):
        assert_tables_match(keys, pairs, okeys, opairs)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_nccl_ranks(tmp_path):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "nccl_rank.py"), str(r), "2", str(port), str(tmp_path)], cwd=ROOT, env=env) for r in range(2)]
    assert [p.wait(timeout=300) for p in procs] == [0, 0]
    rec = trace.generate(trace.config("c3", 400_000))
    okeys, opairs = O.build_pair_table(rec)
    n = 4000
    start = np.arange(n, dtype=np.uint64) * 100 + 1000
    dur = np.full(n, 60, dtype=np.uint64)
    tenant = 1 + (np.arange(n) % 2)
    tenant[3], dur[3] = 0, 100 * n
    rec2 = pack_records(tenant, np.ones((n, 3)), np.ones((n, 3)) * 32, np.zeros(n), tenant, np.zeros(n, bool), start, start + dur)
    skeys, spairs = O.build_pair_table(rec2, key_mode=O.KEY_TYPE)
    for r in range(2):
        d = np.load(tmp_path / f"rank{r}.npz")
        assert_tables_match(d["keys"], d["pairs"], okeys, opairs)
        # the native driver: same table, bit for bit the one the Python-driven exchanges gave
        assert_tables_match(d["nkeys"], d["npairs"], okeys, opairs)
        assert d["nkeys"].tobytes() == d["keys"].tobytes() and d["npairs"].tobytes() == d["pairs"].tobytes()
        assert_tables_match(d["skeys"], d["spairs"], skeys, spairs)
        # ... and the one with the bulk exchanges on NCCL instead of peer memory
        assert d["ckeys"].tobytes() == d["keys"].tobytes() and d["cpairs"].tobytes() == d["pairs"].tobytes()
        print("peer memory:", bool(d["peer_memory"]))
        assert bool(d["two_stage_ok"])  # two key ranges per rank, the first stored while the second is reduced: the same bytes
        assert int(d["bad_status"]) == 3  # KS_ERR_RECORD on BOTH ranks, although only the last rank's window held the bad record
        assert_tables_match(d["t3keys"], d["t3pairs"], *O.build_pair_table(rec[:3]))  # ragged windows
        assert_tables_match(d["t1keys"], d["t1pairs"], *O.build_pair_table(rec[:1]))  # an empty window on the second rank


@pytest.mark.parametrize("cfg,n,key_type", [("c1", 60_000, False), ("c2", 300_000, True), ("c1", 0, False)])
def test_native_driver_single_rank(cfg, n, key_type):
    """ks_mg_build with a communicator of one rank: every phase and exchange of the native driver except the halo."""
    rec = trace.generate(trace.config(cfg, max(n, 4096)))[:n]
    okeys, opairs = O.build_pair_table(rec, key_mode=O.KEY_TYPE if key_type else O.KEY_SHAPE)
    with PairTableBuilder(device=0) as b:
        session = parallel.NativeSession(b)
        window = torch.from_numpy(rec.view(np.uint8).reshape(-1).copy()).cuda()
        torch.cuda.synchronize()
        for _ in range(2):
            keys, pairs = session.build(window, key_type=key_type)
            assert_tables_match(keys, pairs, okeys, opairs)
        session.close()


@pytest.mark.parametrize("stages,refine", [("2", "0"), ("4", "0"), ("4", "1")])
def test_native_driver_in_stages_single_rank(stages, refine, monkeypatch):
    """The staged build (every rank owns several key ranges, reduced one after the other, each sorted over the bits of its
    own width, their rows placed in key-range order) with one rank: no peers to copy to, everything else as on eight GPUs."""
    monkeypatch.setenv("KS_MG_STAGES", stages)
    monkeypatch.setenv("KS_MG_REFINE", refine)  # 1: the cuts between key ranges placed inside histogram bins (equal sample counts)
    with PairTableBuilder(device=0) as b:
        session = parallel.NativeSession(b)
        for cfg, n, key_type in (("c3", 400_000, False), ("c4", 500_000, False), ("c2", 300_000, True), ("c1", 3, False), ("c1", 0, False)):
            rec = trace.generate(trace.config(cfg, max(n, 4096)))[:n]
            okeys, opairs = O.build_pair_table(rec, key_mode=O.KEY_TYPE if key_type else O.KEY_SHAPE)
            window = _window(rec)
            for _ in range(2):  # the second call knows the last table's size
                keys, pairs = session.build(window, key_type=key_type)
                assert_tables_match(keys, pairs, okeys, opairs)
        # ... and the same handle without stages afterwards
        monkeypatch.delenv("KS_MG_STAGES")
        rec = trace.generate(trace.config("c3", 200_000))
        keys, pairs = session.build(_window(rec))
        assert_tables_match(keys, pairs, *O.build_pair_table(rec))
        session.close()


def _window(rec):
    t = torch.from_numpy(rec.view(np.uint8).reshape(-1).copy()).cuda()
    torch.cuda.synchronize()
    return t


def test_native_driver_statuses_and_recovery():
    """Device-detected errors come back as status codes through the exchange headers; the session stays usable."""
    from kernel_scheduling_b200 import _lib

    rec = trace.generate(trace.config("c1", 5000))
    with PairTableBuilder(device=0) as b:
        session = parallel.NativeSession(b)
        bad = rec.copy()
        bad["end_ns"][17] = bad["start_ns"][17] - 1
        with pytest.raises(_lib.KsError) as e:
            session.build(_window(bad))
        assert e.value.status == _lib.ERR_RECORD
        with pytest.raises(_lib.KsError) as e:
            session.build(_window(trace.shuffled(rec)))
        assert e.value.status == _lib.ERR_NOT_ORDERED
        keys, pairs = session.build(_window(rec))
        assert_tables_match(keys, pairs, *O.build_pair_table(rec))
        session.close()
        # without a communicator the call is refused, not run
        with pytest.raises(_lib.KsError) as e:
            session.build(_window(rec))
        assert e.value.status == _lib.ERR_ARG


def test_native_driver_grows_key_block_and_sample_stream():
    # more distinct keys than the first exchange holds by default (4,096): the build starts over with a larger block
    n = 12_000
    start = np.arange(n, dtype=np.uint64) * 50 + 1000
    names = np.arange(n) % 6000
    tenant = np.arange(n) % 2
    rec = pack_records(names, np.ones((n, 3)), np.ones((n, 3)) * 64, np.zeros(n), tenant, (np.arange(n) % 5) == 0, start, start + np.uint64(120))
    # and eight tenants with long launches: far more overlapping pairs than twice the records (the first guess)
    m = 40_000
    start2 = np.arange(m, dtype=np.uint64) * 100 + 1000
    rec2 = pack_records(np.arange(m) % 50, np.ones((m, 3)), np.ones((m, 3)) * 64, np.zeros(m), np.arange(m) % 8, np.zeros(m, bool), start2, start2 + np.uint64(1500))
    with PairTableBuilder(device=0) as b:
        session = parallel.NativeSession(b)
        sizes = []
        for r in (rec, rec2):
            okeys, opairs = O.build_pair_table(r)
            keys, pairs = session.build(_window(r))
            assert_tables_match(keys, pairs, okeys, opairs)
            sizes.append((len(keys), int(pairs["count"].sum())))
        assert sizes[0][0] > 4096 and sizes[1][1] > 2 * (m + 4096)  # the cases are what they claim to be
        session.close()
