"""Generates the golden vectors under tests/golden/ by RUNNING THE REFERENCE'S OWN CODE where it lies.

    python tests/golden/make_golden.py          (needs the reference tree; run in the build container)

  postprocess_cases.json   inputs (two start_ns columns) and the exact stdout of scheduler/postprocess.py
  combine_in_*.csv / combine_out_*.csv   inputs and outputs of postprocess/profile_postprocess.py's CLI
  function_base.tsv        symbol -> ncu_function_base(symbol), from oracle/_ref/ref_function_base
  pair_table_small.npz     the main path (no reference implementation exists for it): seeded traces of a few thousand launches
                           and their tables from the O(n^2) restatement that uses numpy.median (SHAPE and TYPE keys)
The vectors are committed; the tests never read the reference tree.
"""
import json
import os
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np
import pandas as pd

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
REF = Path(os.environ.get("KS_REFERENCE_DIR") or ROOT.parent / "reference")  # the reference checkout beside this repository
TIMING_COLS = ["kernel_id", "kernel_us", "prefetch_us", "prefetch_to_kernel_gap_us", "hook_tag", "prefetch_bytes", "prefetched_tensors", "args_check",
               "kernel_name", "start_ns", "end_ns", "batch_id", "batch_size", "batch_pos", "block", "model", "grid"]


def timing_frame(start_ns, model):
    n = len(start_ns)
    return pd.DataFrame({
        "kernel_id": np.arange(n), "kernel_us": np.full(n, 12.5), "prefetch_us": [""] * n, "prefetch_to_kernel_gap_us": [""] * n,
        "hook_tag": ["unknown"] * n, "prefetch_bytes": [0] * n, "prefetched_tensors": [""] * n, "args_check": ["-"] * n,
        "kernel_name": ["sleep_kernel"] * n, "start_ns": start_ns, "end_ns": np.asarray(start_ns) + 12500, "batch_id": np.arange(n) + 1,
        "batch_size": [1] * n, "batch_pos": [0] * n, "block": ["(128, 1, 1)"] * n, "model": [model] * n, "grid": ["(16, 1, 1)"] * n})[TIMING_COLS]


def run_postprocess(s1, s2):
    with tempfile.TemporaryDirectory() as d:
        a, b = os.path.join(d, "a.tsv"), os.path.join(d, "b.tsv")
        timing_frame(s1, "qwen").to_csv(a, sep="\t", index=False)
        timing_frame(s2, "whisper").to_csv(b, sep="\t", index=False)
        r = subprocess.run([sys.executable, str(REF / "scheduler" / "postprocess.py"), a, b], capture_output=True, text=True)
        return r.returncode, r.stdout, ("AssertionError" in r.stderr)


def postprocess_cases():
    rng = np.random.default_rng(42)
    cases = []
    base = 1_000_000_000_000
    inputs = [
        ("small_example", np.arange(1000, 5001, 1000), np.array([2000, 4000, 6000])),
        ("disjoint", base + np.arange(0, 50) * 7919, base + np.arange(0, 40) * 7919 + 3),
        ("empty_second", base + np.arange(0, 10) * 100, np.array([], dtype=np.int64)),
    ]
    pool = base + rng.choice(1_000_000, 700, replace=False) * 1000
    s1 = rng.permutation(pool[:400])
    s2 = rng.permutation(np.concatenate([pool[300:], ]))
    inputs.append(("random_overlap_100", s1, s2))
    inputs.append(("duplicate_in_first", np.array([5, 6, 6, 7]) + base, np.array([6, 9]) + base))
    inputs.append(("duplicate_in_second", np.array([5, 6, 7]) + base, np.array([6, 9, 9]) + base))
    for name, a, b in inputs:
        rc, out, asserted = run_postprocess(np.asarray(a, dtype=np.int64), np.asarray(b, dtype=np.int64))
        cases.append({"name": name, "start1": [int(x) for x in a], "start2": [int(x) for x in b], "returncode": rc, "stdout": out, "assertion": asserted})
        print(name, rc, out.strip().splitlines()[-1] if out.strip() else "", asserted)
    (HERE / "postprocess_cases.json").write_text(json.dumps(cases, indent=0))


def combine_cases():
    rng = np.random.default_rng(7)
    labels = ["Duration/Wave (us)", "Blocks/Wave", "SM Util %", "Achieved Occ %", "IPC (active)", "L2 Throughput %", "L2 Hit Rate %", "DRAM BW Util %"]
    # case 0: the four-row example; case 1: a few hundred pooled rows with empty cells, a Grid column and the excluded columns
    frames = []
    f0 = pd.DataFrame({"Kernel": ["k1", "k1", "k2", "k2"], "Block": ["(128, 1, 1)"] * 4, "Launches": [3, 1, 2, 2]})
    for j, lab in enumerate(labels):
        f0[lab] = [1.0, 5.0, 2.0, 4.0]
        f0[lab + " std"] = [0.1, 0.0, 0.2, 0.2]
    f0.loc[3, "SM Util %"] = np.nan
    frames.append(f0)
    n = 400
    kern = rng.choice([f"kernel_{i}" for i in range(37)], n)
    block = rng.choice(["(128, 1, 1)", "(256, 1, 1)", "(32, 8, 1)"], n)
    f1 = pd.DataFrame({"Kernel": kern, "Block": block, "Grid": rng.choice(["(1, 1, 1)", "(132, 1, 1)"], n), "Launches": rng.integers(1, 1200, n)})
    for lab in labels + ["Shared Mem Pipe %"]:
        v = rng.normal(50, 20, n)
        v[rng.random(n) < 0.15] = np.nan
        f1[lab] = v
        f1[lab + " std"] = np.abs(rng.normal(1, 0.5, n))
    f1.loc[f1["Kernel"] == "kernel_3", "IPC (active)"] = np.nan  # an all-NaN group
    frames.append(f1)
    for i, f in enumerate(frames):
        src, dst = HERE / f"combine_in_{i}.csv", HERE / f"combine_out_{i}.csv"
        f.to_csv(src, index=False)
        subprocess.run([sys.executable, str(REF / "postprocess" / "profile_postprocess.py"), str(src), str(dst)], check=True)
        print("combine", i, len(f), "->", len(pd.read_csv(dst)))


def function_base_cases():
    sys.path.insert(0, str(ROOT))
    from oracle import build_ref

    build_ref.build()
    with tempfile.TemporaryDirectory() as d:
        obj = os.path.join(d, "c.o")
        subprocess.run(["g++", "-std=c++17", "-O0", "-c", str(HERE / "symbols_corpus.cpp"), "-o", obj], check=True)
        nm = subprocess.run(["nm", "--defined-only", obj], capture_output=True, text=True, check=True).stdout
    syms = sorted({line.split()[-1] for line in nm.splitlines() if line.split()})
    syms += ["_apply_write_kernel", "triton_poi_fused_add_0", "", "_Znot_a_real_mangled_name", "void at::native::(anonymous namespace)::foo<float>(float*)",
             "ns::f<(1)>(2)>(int)", "operator<", "a b c"]
    r = subprocess.run([str(ROOT / "oracle" / "_ref" / "ref_function_base")], input="\n".join(syms) + "\n", capture_output=True, text=True, check=True)
    (HERE / "function_base.tsv").write_text(r.stdout)
    print("function_base", len(r.stdout.splitlines()), "symbols")


def ncu_pool_case():
    """Per-launch label values of real Nsight Compute reports, extracted with the reference script's own helpers, and the
    summary CSV the reference script writes for the same reports (profiling/ncu-bench/ncu_summary.py).  The reports are
    named in KS_NCU_REPORTS (os.pathsep separated); without it the committed fixtures are left alone."""
    reports = [p for p in os.environ.get("KS_NCU_REPORTS", "").split(os.pathsep) if p]
    if not reports:
        print("ncu_pool_case: KS_NCU_REPORTS not set, fixtures unchanged")
        return
    import importlib.util
    import math

    script = REF / "profiling" / "ncu-bench" / "ncu_summary.py"
    spec = importlib.util.spec_from_file_location("ref_ncu_summary", script)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    ncu_report = ref.import_ncu_report(None)
    labels = [ref.RATIO_LABEL, ref.BPW_LABEL] + list(ref.METRICS)
    rows = []
    for path in reports:
        ctx = ncu_report.load_report(path)
        for i in range(ctx.num_ranges()):
            rng = ctx.range_by_idx(i)
            for j in range(rng.num_actions()):
                action = rng.action_by_idx(j)
                row = {"Kernel": action.name(), "Block": ref.fmt_dims(ref.get_dims(action, "block"))}
                dur_us = ref.get_value(action, ref.DURATION_METRIC)
                grid = ref.get_dims(action, "grid")
                waves = ref.get_waves(action, grid, None)
                grid_total = ref.get_value(action, "launch__grid_size")
                if grid_total is None and grid:
                    grid_total = math.prod(grid)
                row["duration_us"], row["waves"], row["grid_total"] = dur_us, waves, grid_total
                for label, candidates in ref.METRICS.items():
                    for metric in candidates:
                        v = ref.get_value(action, metric)
                        if v is not None:
                            row[label] = v
                            break
                rows.append(row)
    frame = pd.DataFrame(rows, columns=["Kernel", "Block", "duration_us", "waves", "grid_total"] + list(ref.METRICS))
    frame.to_csv(HERE / "ncu_launches.csv", index=False, float_format="%.17g")
    subprocess.run([sys.executable, str(script), *reports, "--csv", str(HERE / "ncu_summary_ref.csv")], check=True, capture_output=True)
    print(f"ncu_pool_case: {len(frame)} launches, labels {labels}")


def pair_table_case():
    """The interval join + slowdown statistics have no reference implementation to run.  Their fixture is the table the
    quadratic pure-Python restatement gives (the slowest and plainest statement of the definitions), stored with its input."""
    sys.path.insert(0, str(ROOT))
    from kernel_scheduling_b200 import trace
    from oracle import pair_table_oracle as O

    out = {}
    for tag, cfg, n, mode in (("c1", "c1", 2500, O.KEY_SHAPE), ("c3", "c3", 2000, O.KEY_SHAPE), ("c2type", "c2", 2000, O.KEY_TYPE)):
        spec = trace.config(cfg, n)
        for t in spec.tenants:
            t.n_keys = min(t.n_keys, 40)  # few keys: rows with many samples, even and odd counts
        rec = trace.generate(spec, interleave_solo=(tag == "c3"))
        keys, pairs = O.build_pair_table_bruteforce(rec, key_mode=mode)  # dicts of columns
        out[f"{tag}.records"], out[f"{tag}.mode"] = rec, np.int64(mode)
        for c, v in keys.items():
            out[f"{tag}.keys.{c}"] = v
        for c, v in pairs.items():
            out[f"{tag}.pairs.{c}"] = v
        print(f"pair_table_case {tag}: {len(rec)} records, {len(keys['key'])} keys, {len(pairs['count'])} rows, {int(pairs['count'].sum())} pairs, "
              f"largest row {int(pairs['count'].max())}")
    np.savez_compressed(HERE / "pair_table_small.npz", **out)


if __name__ == "__main__":
    pair_table_case()
    postprocess_cases()
    combine_cases()
    function_base_cases()
    ncu_pool_case()
