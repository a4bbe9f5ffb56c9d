"""CPU: ingest of agent timing logs, the TSV emit, and acceptance of the emitted files by the reference's own loader."""
import os
import re
import subprocess
import time

import numpy as np
import pandas as pd
import pytest

from kernel_scheduling_b200 import make_pair_eff as M
from kernel_scheduling_b200 import trace
from kernel_scheduling_b200.records import KEY_ROW_DTYPE, PAIR_ROW_DTYPE
from oracle import pair_table_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DAEMON = os.path.join(ROOT, "oracle", "_ref", "scheduler_daemon")


def oracle_tables_as_rows(rec, key_mode):
    """Oracle columns -> the structured arrays the library returns (so the emit can be tested without a GPU)."""
    k, p = O.build_pair_table(rec, key_mode=key_mode)
    keys = np.zeros(len(k["key"]), dtype=KEY_ROW_DTYPE)
    for c in ("key", "name_id", "grid", "block", "smem", "tenant", "launches", "solo_launches", "solo_ns"):
        keys[c] = k[c]
    pairs = np.zeros(len(p["count"]), dtype=PAIR_ROW_DTYPE)
    for c in p:
        pairs[c] = p[c]
    return keys, pairs


def synthetic_timing_frames(n=3000):
    """Two co-run and two solo agent logs with the 17 columns of scheduler/agent.cpp:692."""
    rec = trace.generate(trace.config("c1", n))
    solo = (rec["smem_word"] & (1 << 23)) != 0
    ten = rec["smem_word"] >> 24
    frames = {}
    for t, model in enumerate(("qwen", "whisper")):
        for s in (False, True):
            r = rec[(ten == t) & (solo == s)]
            m = len(r)
            frames[(model, s)] = pd.DataFrame({
                "kernel_id": np.arange(m), "kernel_us": (r["end_ns"] - r["start_ns"]) / 1e3, "prefetch_us": [""] * m, "prefetch_to_kernel_gap_us": [""] * m,
                "hook_tag": ["unknown"] * m, "prefetch_bytes": [0] * m, "prefetched_tensors": [""] * m, "args_check": ["-"] * m,
                "kernel_name": [f"void ns::kernel_{i}<float>(float*)" for i in r["name_id"]], "start_ns": r["start_ns"], "end_ns": r["end_ns"].astype("float64"),
                "batch_id": np.arange(m) + 1, "batch_size": [1] * m, "batch_pos": [0] * m,
                "block": [f"({b[0]}, {b[1]}, {b[2]})" for b in r["block"]], "model": [model] * m, "grid": [f"({g[0]}, {g[1]}, {g[2]})" for g in r["grid"]]})
    return rec, frames


def test_ingest_builds_equivalent_records():
    rec, frames = synthetic_timing_frames()
    f = frames[("qwen", False)].copy()
    f.loc[5, "end_ns"] = np.nan  # a launch whose completion callback was never seen is dropped
    ing = M.TraceIngest()
    parts = [ing.records(f, False), ing.records(frames[("whisper", False)], False), ing.records(frames[("qwen", True)], True), ing.records(frames[("whisper", True)], True)]
    got = np.concatenate(parts)
    assert len(got) == len(rec) - 1 and ing.models == ["qwen", "whisper"]
    assert all(re.fullmatch(r"kernel_\d+", n) for n in ing.names)
    # same table as the original records up to the renumbering of names (and smem, which the logs do not carry)
    ref = rec.copy()
    ref["smem_word"] &= np.uint32(0xFF800000)
    _, p_got = O.build_pair_table(got)
    _, p_ref = O.build_pair_table(ref[np.isin(np.arange(len(ref)), np.flatnonzero((ref["smem_word"] >> 24 == 0) & ((ref["smem_word"] & (1 << 23)) == 0))[5:6], invert=True)])
    assert sorted(p_got["count"].tolist()) == sorted(p_ref["count"].tolist())


def test_emitted_tables_have_the_daemon_columns(tmp_path):
    rec = trace.generate(trace.config("c1", 4000))
    names = [f"k{i}" for i in range(int(rec["name_id"].max()) + 1)]
    tables = [(*oracle_tables_as_rows(rec, O.KEY_SHAPE), False), (*oracle_tables_as_rows(rec, O.KEY_TYPE), True)]
    us, eff = M.write_tables(str(tmp_path), tables, names, ["qwen", "whisper"])
    du, de = pd.read_csv(us, sep="\t"), pd.read_csv(eff, sep="\t")
    assert list(du.columns[:6]) == ["model", "kernel", "block", "grid", "solo_us", "launches"]
    assert list(de.columns[:10]) == ["model_a", "kernel_a", "block_a", "grid_a", "model_b", "kernel_b", "block_b", "grid_b", "efficiency", "gangs"]
    assert ((de["grid_a"] == "*") == (de["grid_b"] == "*")).all()  # both grids or neither (scheduler_daemon.cpp:240)
    assert (de["model_a"] == "qwen").all() and (de["model_b"] == "whisper").all()
    keys, pairs, _ = tables[0]
    n_shape = int(np.isfinite(pairs["efficiency"]).sum())
    assert (de["grid_a"] != "*").sum() == n_shape
    row = de[de["grid_a"] != "*"].iloc[0]
    assert float(row["efficiency"]) == pairs["efficiency"][np.isfinite(pairs["efficiency"])][0]  # repr() round-trips doubles


@pytest.mark.skipif(not os.path.exists(DAEMON), reason="the reference daemon is only built where the reference tree is present")
def test_reference_daemon_loads_the_emitted_tables(tmp_path):
    rec = trace.generate(trace.config("c1", 4000))
    names = [f"k{i}" for i in range(int(rec["name_id"].max()) + 1)]
    tables = [(*oracle_tables_as_rows(rec, O.KEY_SHAPE), False), (*oracle_tables_as_rows(rec, O.KEY_TYPE), True)]
    us, eff = M.write_tables(str(tmp_path), tables, names, ["qwen", "whisper"])
    env = dict(os.environ, SCHED_MODE="eff", SCHED_PAIR_EFF_FILE=eff, SCHED_KERNEL_US_FILE=us, SCHED_LOG="off", SCHED_LOG_DIR=str(tmp_path))
    proc = subprocess.Popen([DAEMON], env=env, stderr=subprocess.PIPE, stdout=subprocess.DEVNULL, text=True)
    line = ""
    try:
        deadline = time.time() + 20
        while time.time() < deadline:
            out = proc.stderr.readline()
            if not out:
                break
            if "type-pair rows" in out:
                line = out
                break
    finally:
        proc.terminate()
        try:
            proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            proc.kill()
    m = re.search(r"(\d+) type-pair rows, (\d+) shape-pair rows.*SCHED_KERNEL_US_FILE: (\d+) rows", line)
    assert m, f"the daemon did not report the tables: {line!r}"
    n_type = int(np.isfinite(tables[1][1]["efficiency"]).sum())
    n_shape = int(np.isfinite(tables[0][1]["efficiency"]).sum())
    n_us = int(np.isfinite(tables[0][0]["solo_ns"]).sum()) + int(np.isfinite(tables[1][0]["solo_ns"]).sum())
    assert (int(m.group(1)), int(m.group(2)), int(m.group(3))) == (n_type, n_shape, n_us)
    assert "WARNING" not in line


def test_pairprof_labels_in_the_pandas_ingest():
    """The host-side meaning of a pairprof log: alone* = solo sample, gang* = co-run launch, not mentioned = dropped."""
    from kernel_scheduling_b200 import make_pair_eff as M

    _, frames = synthetic_timing_frames(600)
    f = frames[("qwen", False)].copy().reset_index(drop=True)
    f["kernel_id"] = np.arange(len(f)) + 3
    log = pd.DataFrame({"batch_id": 1, "kind": ["alone", "gang_profile", "alone_other_waits", "gang_filler", "alone"], "pid": [5, 5, 5, 5, 6],
                        "kernel_id": [3, 4, 5, 6, 7], "model": "qwen", "kernel": "k", "block": "1,1,1", "rep": "", "grid": "1,1,1"})
    rec = M.TraceIngest().records(f, False, pairprof=log, pid=5)
    assert len(rec) == 4  # kernel_id 7 belongs to another process, the rest of the file is not mentioned
    assert list((rec["smem_word"] >> 23) & 1) == [1, 0, 1, 0]
    assert list(rec["start_ns"]) == list(f["start_ns"][:4])
    assert M.agent_pid("/x/agent_123_timing.tsv") == 123 and M.agent_pid("a.tsv") is None


def test_pair_table_in_shared_memory_python_and_c_readers(tmp_path):
    """Publish the SHAPE and TYPE tables into a POSIX segment; read them back with the Python reader and with a C99 program
    that uses the header alone; the daemon's fallback rule (scheduler_daemon.cpp:269-274) on both."""
    import subprocess

    from kernel_scheduling_b200 import pair_table_shm as PT

    rec = trace.generate(trace.config("c1", 4000))
    shape = oracle_tables_as_rows(rec, O.KEY_SHAPE)
    typ = oracle_tables_as_rows(rec, O.KEY_TYPE)
    names = [f"kernel_{i}" for i in range(int(rec["name_id"].max()) + 1)]
    models = ["qwen", "whisper"]
    name = f"/ks_pairtab_test_{os.getpid()}"
    try:
        nbytes = PT.publish(shape, typ, names, models, name=name, generation=7)
        assert nbytes == os.path.getsize("/dev/shm" + name) and not os.path.exists("/dev/shm" + name + ".tmp")
        # the host key function is the oracle's hash
        k0 = shape[0][0]
        assert PT.kernel_key(int(k0["name_id"]), k0["grid"], k0["block"], int(k0["tenant"]), smem=int(k0["smem"])) == int(k0["key"])
        type_of_shape = {int(r["key"]): PT.kernel_key(int(r["name_id"]), (0, 0, 0), r["block"], int(r["tenant"]), type_key=True) for r in shape[0]}
        assert set(type_of_shape.values()) == {int(k) for k in typ[0]["key"]}
        with PT.Attached(name) as seg:
            assert seg.generation == 7 and seg.names == names and seg.models == models
            assert len(seg.shape.keys) == len(shape[0]) and len(seg.shape.vals) == len(shape[1]) and len(seg.type.vals) == len(typ[1])
            for table, (keys, pairs) in ((seg.shape, shape), (seg.type, typ)):
                for p in pairs[:: max(1, len(pairs) // 300)]:
                    for x, y in ((p["key_a"], p["key_b"]), (p["key_b"], p["key_a"])):  # either order
                        v = table.find_pair(int(x), int(y))
                        assert v is not None and v[1] == int(p["count"])
                        assert (np.isnan(v[0]) and np.isnan(p["efficiency"])) or v[0] == np.float32(p["efficiency"])
                assert table.find_pair(int(keys["key"][0]), int(keys["key"][0])) is None  # same tenant: no such row
                assert table.find_key(12345) == -1
            # the fallback: a shape pair seen fewer than min_gangs times answers with its type row
            queries, want = [], []
            min_gangs = 3
            for p in shape[1][:: max(1, len(shape[1]) // 200)]:
                ta, tb = type_of_shape[int(p["key_a"])], type_of_shape[int(p["key_b"])]
                v = seg.lookup_eff(int(p["key_a"]), int(p["key_b"]), ta, tb, min_gangs)
                trow = seg.type.find_pair(ta, tb)
                assert trow is not None
                expect = (np.float32(p["efficiency"]), int(p["count"])) if int(p["count"]) >= min_gangs else trow
                assert v[1] == expect[1] and (v[0] == expect[0] or (np.isnan(v[0]) and np.isnan(expect[0])))
                queries.append(f"{int(p['key_a'])} {int(p['key_b'])} {ta} {tb}")
                kus = seg.kernel_us(int(p["key_a"]), ta)
                want.append((int(np.float32(v[0]).view(np.uint32)), v[1], int(np.float64(kus).view(np.uint64))))
            queries.append("1 2 3 4")
            want.append((-1, -1, int(np.float64(np.nan).view(np.uint64))))
        exe = str(tmp_path / "pairtab_reader")
        here = os.path.dirname(os.path.abspath(__file__))
        subprocess.run(["gcc", "-std=c99", "-O1", "-Wall", "-Werror", "-D_POSIX_C_SOURCE=200809L", "-o", exe, os.path.join(here, "pairtab_reader.c"), "-lrt"], check=True)
        out = subprocess.run([exe, name, str(min_gangs)], input="\n".join(queries) + "\n", capture_output=True, text=True, check=True).stdout.split("\n")
        assert out[0].split() == ["7", str(len(shape[0])), str(len(shape[1])), str(len(typ[0])), str(len(typ[1]))]
        got = [tuple(int(x) for x in line.split()) for line in out[1: 1 + len(want)]]
        assert got == want
        # a second publish replaces the segment atomically; rows out of order are refused
        PT.publish(shape, typ, names, models, name=name, generation=8)
        with PT.Attached(name) as seg:
            assert seg.generation == 8
        from kernel_scheduling_b200 import _lib

        with pytest.raises(_lib.KsError):
            PT.publish((shape[0], shape[1][::-1]), typ, names, models, name=name)
    finally:
        PT.unlink(name)
    assert not os.path.exists("/dev/shm" + name)
