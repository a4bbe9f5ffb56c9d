"""GPU: the reference-facing entry points against the reference's own outputs (golden vectors)."""
import contextlib
import io
import json
import os

import numpy as np
import pandas as pd
import pytest

from kernel_scheduling_b200 import make_pair_eff as M
from kernel_scheduling_b200 import postprocess, profile_postprocess
from oracle import pair_table_oracle as O
from tests.test_host_logic import oracle_tables_as_rows, synthetic_timing_frames
from tests.golden.make_golden import timing_frame

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_postprocess_cli_prints_what_the_reference_prints(tmp_path):
    for c in json.load(open(os.path.join(GOLDEN, "postprocess_cases.json"))):
        a, b = str(tmp_path / "a.tsv"), str(tmp_path / "b.tsv")
        timing_frame(np.array(c["start1"], dtype=np.int64), "qwen").to_csv(a, sep="\t", index=False)
        timing_frame(np.array(c["start2"], dtype=np.int64), "whisper").to_csv(b, sep="\t", index=False)
        buf = io.StringIO()
        if c["assertion"]:
            with pytest.raises(AssertionError), contextlib.redirect_stdout(buf):
                postprocess.main([a, b])
        else:
            with contextlib.redirect_stdout(buf):
                assert postprocess.main([a, b]) == 0
            assert buf.getvalue() == c["stdout"], c["name"]


@pytest.mark.parametrize("case", [0, 1])
def test_combine_duplicates_frame_equals_reference_csv(builder, case, tmp_path):
    df = pd.read_csv(os.path.join(GOLDEN, f"combine_in_{case}.csv"))
    want = pd.read_csv(os.path.join(GOLDEN, f"combine_out_{case}.csv"))
    got = profile_postprocess.combine_duplicates(df, builder)
    assert list(got.columns) == list(want.columns)
    assert got["Kernel"].tolist() == want["Kernel"].tolist() and got["Block"].tolist() == want["Block"].tolist()
    assert got["Launches"].tolist() == want["Launches"].tolist()
    vals = [c for c in want.columns if c not in ("Kernel", "Block", "Launches")]
    assert np.allclose(got[vals].to_numpy(), want[vals].to_numpy(), rtol=1e-12, atol=0, equal_nan=True)
    out = str(tmp_path / "o.csv")
    assert profile_postprocess.main([os.path.join(GOLDEN, f"combine_in_{case}.csv"), out]) == 0
    assert np.allclose(pd.read_csv(out)[vals].to_numpy(), want[vals].to_numpy(), rtol=1e-12, atol=0, equal_nan=True)


def test_make_pair_eff_end_to_end(tmp_path):
    rec, frames = synthetic_timing_frames(5000)
    paths = {}
    for (model, solo), f in frames.items():
        paths[(model, solo)] = str(tmp_path / f"{model}_{int(solo)}.tsv")
        f.to_csv(paths[(model, solo)], sep="\t", index=False)
    out = str(tmp_path / "out")
    assert M.main(["--corun", paths[("qwen", False)], paths[("whisper", False)], "--solo", paths[("qwen", True)], paths[("whisper", True)], "--out-dir", out]) == 0
    # expected files: the same ingest, tables from the oracle, same writer
    ing = M.TraceIngest()
    parts = [ing.records(pd.read_csv(paths[k], sep="\t"), k[1]) for k in (("qwen", False), ("whisper", False), ("qwen", True), ("whisper", True))]
    r2 = np.concatenate(parts)
    tables = [(*oracle_tables_as_rows(r2, O.KEY_SHAPE), False), (*oracle_tables_as_rows(r2, O.KEY_TYPE), True)]
    want = str(tmp_path / "want")
    M.write_tables(want, tables, ing.names, ing.models)
    for name in ("kernel_us.tsv",):
        assert open(os.path.join(out, name)).read() == open(os.path.join(want, name)).read()
    got_eff, want_eff = pd.read_csv(os.path.join(out, "pair_eff.tsv"), sep="\t"), pd.read_csv(os.path.join(want, "pair_eff.tsv"), sep="\t")
    exact = [c for c in got_eff.columns if "mean" not in c]
    assert got_eff[exact].equals(want_eff[exact])
    assert np.allclose(got_eff[["slowdown_mean_a", "slowdown_mean_b"]].to_numpy(), want_eff[["slowdown_mean_a", "slowdown_mean_b"]].to_numpy(), rtol=1e-6, atol=0)


def test_device_tsv_parse_equals_pandas_ingest(builder, tmp_path):
    rec, frames = synthetic_timing_frames(6000)
    f = frames[("qwen", False)].copy()
    f.loc[[5, 77], "end_ns"] = np.nan  # launches whose completion callback was never seen: dropped by both routes
    f["block"] = [b.replace("(", "").replace(")", "").replace(" ", "") if i % 2 else b for i, b in enumerate(f["block"])]  # "x,y,z" spelling
    texts = {}
    for key, frame in ((("qwen", False), f), (("whisper", False), frames[("whisper", False)]), (("qwen", True), frames[("qwen", True)])):
        p = str(tmp_path / f"{key[0]}_{int(key[1])}.tsv")
        frame.to_csv(p, sep="\t", index=False)
        texts[key] = (p, frame)
    ing_a, ing_b = M.TraceIngest(), M.TraceIngest()
    for key, (p, frame) in texts.items():
        want = ing_a.records(pd.read_csv(p, sep="\t"), key[1])
        got = M.records_from_log(ing_b, builder, p, key[1])
        assert len(got) == len(want) and got.tobytes() == want.tobytes(), key
    assert ing_a.names == ing_b.names and ing_a.models == ing_b.models
    # no trailing newline, CRLF line ends, an empty file body
    raw = open(texts[("whisper", False)][0], "rb").read()
    want = ing_a.records(texts[("whisper", False)][1], False)
    assert M.records_from_log(ing_b, builder, raw.rstrip(b"\n"), False).tobytes() == want.tobytes()
    assert M.records_from_log(ing_b, builder, raw.replace(b"\n", b"\r\n"), False).tobytes() == want.tobytes()
    assert len(M.records_from_log(ing_b, builder, raw.split(b"\n")[0] + b"\n", False)) == 0


def test_device_tsv_parse_numbers_models_over_the_kept_rows_only(builder, tmp_path):
    """A file with two models whose second model first shows up on a row that is DROPPED (no end_ns): the tenants must be
    numbered over the rows that are kept, as the pandas route numbers them -- which launch is side a depends on it."""
    rec, frames = synthetic_timing_frames(3000)
    a, b = frames[("qwen", False)].copy(), frames[("whisper", False)].copy()
    both = pd.concat([b.iloc[:1], a, b.iloc[1:]]).reset_index(drop=True)  # row 0: the other model ...
    both["end_ns"] = both["end_ns"].astype(float)
    both.loc[0, "end_ns"] = np.nan                                        # ... on a row without a completion time
    p = str(tmp_path / "two_models.tsv")
    both.to_csv(p, sep="\t", index=False)
    ing_a, ing_b = M.TraceIngest(), M.TraceIngest()
    want = ing_a.records(pd.read_csv(p, sep="\t"), False)
    got = M.records_from_log(ing_b, builder, p, False)
    assert ing_a.models == ing_b.models and ing_a.models[0] == "qwen"
    assert len(got) == len(want) == len(both) - 1 and got.tobytes() == want.tobytes()


def _one_run_with_pairprof_log(n, tmp_path):
    """One profiling run as the reference leaves it on disk: an agent log per process holding ALL its launches (solo and
    gang, numbered by kernel_id) and the daemon's log that says which was which (pairprof_daemon.cpp:266, :317-318)."""
    rec, frames = synthetic_timing_frames(n)
    pids = {"qwen": 4101, "whisper": 4102}
    rng = np.random.default_rng(11)
    agent_paths, log_rows = {}, []
    for model, pid in pids.items():
        both = pd.concat([frames[(model, False)].assign(_solo=False), frames[(model, True)].assign(_solo=True)]).sort_values("start_ns", kind="stable").reset_index(drop=True)
        both["kernel_id"] = np.arange(len(both)) + 7  # the agent's running number does not start at 0 after the warm-up
        unlisted = rng.random(len(both)) < 0.05        # launches the profiler never registered (warm-up): dropped
        for i, row in both.iterrows():
            if unlisted[i]:
                continue
            kind = ("alone" if i % 3 else "alone_other_waits") if row["_solo"] else ("gang_profile" if i % 2 else "gang_filler")
            block = row["block"].strip("()").replace(" ", "")
            log_rows.append((i + 1, kind, pid, int(row["kernel_id"]), model, "k", block, "1" if kind == "gang_profile" else "", "1,1,1"))
            # a row of ANOTHER process with the same kernel_id and the opposite kind must not label this launch
            if i % 50 == 0:
                log_rows.append((i + 1, "gang_filler" if row["_solo"] else "alone", 9999, int(row["kernel_id"]), model, "k", block, "", "1,1,1"))
        p = str(tmp_path / f"agent_{pid}_timing.tsv")
        both.drop(columns="_solo").to_csv(p, sep="\t", index=False)
        agent_paths[model] = p
    log = pd.DataFrame(log_rows, columns=["batch_id", "kind", "pid", "kernel_id", "model", "kernel", "block", "rep", "grid"])
    log_path = str(tmp_path / "pairprof_log_77.tsv")
    log.to_csv(log_path, sep="\t", index=False)
    return pids, agent_paths, log_path


def test_pairprof_log_labels_on_the_device_equal_the_pandas_route(builder, tmp_path):
    pids, agent_paths, log_path = _one_run_with_pairprof_log(6000, tmp_path)
    log = pd.read_csv(log_path, sep="\t")
    ing_a, ing_b = M.TraceIngest(), M.TraceIngest()
    total = 0
    for model, pid in pids.items():
        want = ing_a.records(pd.read_csv(agent_paths[model], sep="\t"), False, pairprof=log, pid=pid)
        got = M.records_from_log(ing_b, builder, agent_paths[model], False, pairprof_log=log_path, pid=pid)
        assert len(got) == len(want) and got.tobytes() == want.tobytes(), model
        solo = (want["smem_word"] >> 23) & 1
        assert 0 < solo.sum() < len(want)  # both kinds present
        total += len(want)
    assert ing_a.names == ing_b.names and ing_a.models == ing_b.models
    assert M.agent_pid(agent_paths["qwen"]) == 4101
    # CRLF log, and a log that mentions nothing of this process: every launch is dropped
    raw = open(log_path, "rb").read()
    again = M.records_from_log(M.TraceIngest(), builder, agent_paths["qwen"], False, pairprof_log=raw.replace(b"\n", b"\r\n"), pid=4101)
    assert len(again) == len(ing_a.records(pd.read_csv(agent_paths["qwen"], sep="\t"), False, pairprof=log, pid=4101))
    assert len(M.records_from_log(M.TraceIngest(), builder, agent_paths["qwen"], False, pairprof_log=raw, pid=1)) == 0


def test_make_pair_eff_cli_with_pairprof_log(tmp_path):
    pids, agent_paths, log_path = _one_run_with_pairprof_log(5000, tmp_path)
    out = str(tmp_path / "out")
    assert M.main(["--corun", agent_paths["qwen"], agent_paths["whisper"], "--pairprof-log", log_path, "--out-dir", out]) == 0
    log = pd.read_csv(log_path, sep="\t")
    ing = M.TraceIngest()
    r2 = np.concatenate([ing.records(pd.read_csv(agent_paths[m], sep="\t"), False, pairprof=log, pid=pids[m]) for m in ("qwen", "whisper")])
    tables = [(*oracle_tables_as_rows(r2, O.KEY_SHAPE), False), (*oracle_tables_as_rows(r2, O.KEY_TYPE), True)]
    want = str(tmp_path / "want")
    M.write_tables(want, tables, ing.names, ing.models)
    assert open(os.path.join(out, "kernel_us.tsv")).read() == open(os.path.join(want, "kernel_us.tsv")).read()
    got_eff, want_eff = pd.read_csv(os.path.join(out, "pair_eff.tsv"), sep="\t"), pd.read_csv(os.path.join(want, "pair_eff.tsv"), sep="\t")
    exact = [c for c in got_eff.columns if "mean" not in c]
    assert got_eff[exact].equals(want_eff[exact])


def test_ncu_pooling_on_the_device(builder, tmp_path):
    from kernel_scheduling_b200 import ncu_summary as N
    from tests.test_oracle_golden import _ncu_pool_inputs

    # real reports: the frame the reference script would pool, against the CSV it wrote
    frame, ref = _ncu_pool_inputs()
    got = N.pool_launches(frame, builder)
    assert list(got.columns) == list(ref.columns)
    assert list(got["Kernel"]) == list(ref["Kernel"]) and list(got["Block"]) == list(ref["Block"]) and list(got["Launches"]) == list(ref["Launches"])
    for c in ref.columns[3:]:
        assert np.allclose(got[c].to_numpy(), ref[c].to_numpy(dtype=np.float64), rtol=1e-12, atol=0, equal_nan=True), c
    # CLI round trip
    src, dst = str(tmp_path / "launches.csv"), str(tmp_path / "summary.csv")
    frame.to_csv(src, index=False, float_format="%.17g")
    assert N.main([src, dst]) == 0
    again = pd.read_csv(dst, float_precision="round_trip")
    assert np.allclose(again[ref.columns[3:]].to_numpy(), ref[ref.columns[3:]].to_numpy(dtype=np.float64), rtol=1e-12, atol=0, equal_nan=True)

    # synthetic: thousands of launches, groups from 1 to 4,000 launches, absent cells, a constant column, a large offset
    rng = np.random.default_rng(5)
    rows, cols, groups = 30_000, 6, 200
    gid = np.minimum((rng.pareto(0.7, rows)).astype(np.int64), groups - 1).astype(np.uint32)
    gid[:groups] = np.arange(groups)  # every group has at least one launch
    values = rng.normal(50.0, 10.0, (rows, cols))
    values[:, 1] = 7.25                                  # constant: std exactly 0
    values[:, 2] += 1e9                                  # large mean, small spread
    values[rng.random((rows, cols)) < 0.2] = np.nan      # absent metrics
    values[gid == 3, 4] = np.nan                         # a label no launch of the group has
    launches, mean, std = builder.pool_launches(gid, values, groups)
    ol, om, os_ = O.pool_launches(gid, values, groups)
    assert list(launches) == list(ol)
    assert np.allclose(mean, om, rtol=1e-13, atol=0, equal_nan=True)
    assert np.allclose(std, os_, rtol=1e-9, atol=1e-12, equal_nan=True)  # sample std of n values: conditioning ~ mean / spread
    assert np.all(std[:, 1][~np.isnan(std[:, 1])] == 0.0) and np.isnan(mean[3, 4]) and np.isnan(std[3, 4])


def test_make_pair_eff_publishes_the_tables_in_shared_memory(tmp_path):
    """The segment holds what pair_eff.tsv / kernel_us.tsv hold: every pair row of the files is found by key with the same
    efficiency (as float32) and gangs, every kernel row with the same solo time."""
    from kernel_scheduling_b200 import pair_table_shm as PT

    rec, frames = synthetic_timing_frames(5000)
    paths = {}
    for (model, solo), f in frames.items():
        paths[(model, solo)] = str(tmp_path / f"{model}_{int(solo)}.tsv")
        f.to_csv(paths[(model, solo)], sep="\t", index=False)
    out, name = str(tmp_path / "out"), f"/ks_pairtab_gpu_test_{os.getpid()}"
    try:
        assert M.main(["--corun", paths[("qwen", False)], paths[("whisper", False)], "--solo", paths[("qwen", True)], paths[("whisper", True)],
                       "--out-dir", out, "--publish-shm", name]) == 0
        eff = pd.read_csv(os.path.join(out, "pair_eff.tsv"), sep="\t")
        kus = pd.read_csv(os.path.join(out, "kernel_us.tsv"), sep="\t")
        dims = lambda s: [int(v) for v in str(s).replace("(", "").replace(")", "").split(",")]
        with PT.Attached(name) as seg:
            name_id, tenant = {n: i for i, n in enumerate(seg.names)}, {m: i for i, m in enumerate(seg.models)}

            def key(model, kernel, block, grid):
                is_type = str(grid) == "*"
                return is_type, PT.kernel_key(name_id[kernel], (0, 0, 0) if is_type else dims(grid), dims(block), tenant[model], type_key=is_type)

            assert 100 < len(eff) <= len(seg.shape.vals) + len(seg.type.vals)  # the file leaves out pairs without an efficiency
            for _, r in eff.iloc[:: max(1, len(eff) // 400)].iterrows():
                ta, ka = key(r["model_a"], r["kernel_a"], r["block_a"], r["grid_a"])
                tb, kb = key(r["model_b"], r["kernel_b"], r["block_b"], r["grid_b"])
                assert ta == tb
                v = (seg.type if ta else seg.shape).find_pair(ka, kb)
                assert v is not None and v[1] == int(r["gangs"])
                assert v[0] == np.float32(r["efficiency"]) or (np.isnan(v[0]) and np.isnan(r["efficiency"]))
            for _, r in kus.iloc[:: max(1, len(kus) // 200)].iterrows():
                is_type, k = key(r["model"], r["kernel"], r["block"], r["grid"])
                table = seg.type if is_type else seg.shape
                i = table.find_key(k)
                assert i >= 0 and np.isclose(table.keys["solo_us"][i], float(r["solo_us"]), rtol=1e-12, atol=0)
    finally:
        PT.unlink(name)
