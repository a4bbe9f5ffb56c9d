#!/usr/bin/env python
"""Benchmark of the trace -> interference-table path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c3] [--records R]

A step is one pass of the whole path (decode + hash, grouping sort, interval join, segmented statistics,
tables) over one seeded synthetic trace.  ``value`` is records/s with the trace resident in HBM; ``e2e`` is the
same metric through the public API with HOST buffers (pinned), host<->device copies inside the timed region.
At N > 1 (torchrun, one rank per GPU) every rank takes one time window of the trace.

``--workload c5`` measures the resident table instead (online incremental mode): a step is one window of 65,536 launches
merged into the table, the metric its latency (lower is better); one GPU.

``--impl reference`` times the CPU restatement of the reference's post-processing (oracle/) on the box's host
cores on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "trace records/sec to interference table"
UNIT = "records/s"
CLOCK_LOAD_STEPS = 200  # at most this many untimed steps in front of the warm-up while the clock sampler runs (about 0.2-0.3 s of load)
MIN_TIMED_S = 0.5  # the timed region is at least this long (blocks of K steps are repeated)
CPU_SAMPLE_RECORDS = 20_000_000  # the CPU arm takes a 20 M-record stretch of the workload: several seconds of all host cores per step


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3")
    ap.add_argument("--records", type=int, default=None, help="records per GPU (default: the configuration's own size, capped by --max-records)")
    ap.add_argument("--max-records", type=int, default=100_000_000)
    ap.add_argument("--verify", action="store_true", help="compare the table of the timed workload with the CPU oracle at full size (slow; not part of the default run)")
    ap.add_argument("--windows", type=int, default=10_000, help="--workload c5: windows of 65,536 launches to merge")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--streamed", action="store_true", help="one GPU: the window-by-window build (default for more than 160 M records)")
    ap.add_argument("--window-records", type=int, default=0, help="streamed build: launches per join window (0 = the library's default, 2^26)")
    ap.add_argument("--parts", type=int, default=0, help="streamed build: key ranges (0 = 16)")
    ap.add_argument("--gen-window", type=int, default=125_000_000, help="streamed build: the trace is generated in windows of this many records")
    ap.add_argument("--no-extras", action="store_true", help="skip the first-call, unhinted and per-tenant-runs figures (profiler runs)")
    ap.add_argument("--clock-load-steps", type=int, default=CLOCK_LOAD_STEPS,
                    help="untimed steps in front of the warm-up while the clock sampler starts (0 for profiler runs)")
    ap.add_argument("--mg-driver", default="native", choices=["native", "python"], help="N > 1: who issues the exchanges (the library through NCCL, or torch.distributed)")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def wait_first(self, timeout: float):
        """Returns once nvidia-smi has delivered its first sample (its start-up is over), or after ``timeout`` seconds."""
        t0 = time.perf_counter()
        while self.proc and not self.rows and time.perf_counter() - t0 < timeout:
            time.sleep(0.01)

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def cpu_baseline(workload: str, sample_records: int, rec=None, threads: int = 0):
    """The C restatement of the reference's post-processing (oracle/pair_table_oracle.c) timed on the box's host cores."""
    from kernel_scheduling_b200 import trace
    from oracle import c_oracle

    if rec is None or len(rec) != sample_records:
        rec = trace.generate_fast(trace.config(workload, sample_records))
    cores = threads or c_oracle.host_threads()
    t0 = time.perf_counter()
    _, pairs = c_oracle.build_pair_table(rec, threads=cores)
    dt = time.perf_counter() - t0
    return {"value": len(rec) / dt, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{len(rec)} records of {workload} ({int(pairs['count'].sum())} overlapping pairs, {len(pairs['count'])} rows), C/OpenMP oracle, "
                      f"{cores} threads of {os.cpu_count()} host cores, {dt:.2f} s"}


def run_reference(args, rank, world):
    """The reference arm: the CPU restatement of the path (the reference itself has no installable package and no
    pair-table builder), all host threads, each step a bounded sample of the GPU arm's workload."""
    if rank != 0:
        return
    from kernel_scheduling_b200 import trace

    workload = args.workload
    n = min(CPU_SAMPLE_RECORDS, args.records or CPU_SAMPLE_RECORDS)
    for _ in range(min(args.warmup, 1)):
        cpu_baseline(workload, max(n // 20, 1000))
    rec = trace.generate_fast(trace.config(workload, n))
    vals = [cpu_baseline(workload, n, rec) for _ in range(max(1, min(args.steps, 3)))]
    best = max(vals, key=lambda v: v["value"])
    ms = 1e3 * n / best["value"]
    line = {
        "impl": "reference", "metric": METRIC, "value": best["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": len(vals), "warmup": min(args.warmup, 1),
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int64/f64", "data": "synthetic",
        "config": {"workload": workload_label(workload), "records_per_step": n, "sample": f"{n} records of the same workload per step"},
        "cpu_baseline": best,
        "e2e": {"value": best["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_label(workload: str) -> str:
    """One label for both arms of the benchmark."""
    from kernel_scheduling_b200 import trace

    spec = trace.config(workload)
    return f"{workload}: {len(spec.tenants)} tenants, {sum(t.n_keys for t in spec.tenants)} keys, {spec.n_records} records (synthetic, seeded)"


def run_online(args, rank):
    """--workload c5: the resident table.  A step is one window of 65,536 launches merged into the table; ``value`` is the
    median latency of an update with the window already in device memory over ``--windows`` windows (10,000 as the
    configuration states), ``e2e`` the same for the last 200 windows, which arrive in pinned host memory (their copy to the
    device inside the call).  One GPU: the path does not shard (a table is one sequence of windows)."""
    if rank != 0:
        return
    import torch

    from kernel_scheduling_b200 import online, trace
    from kernel_scheduling_b200.records import RECORD_DTYPE
    from oracle import c_oracle

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the GPU arm")
    per = 65536
    windows = max(args.windows, 300)
    sampler = ClockSampler(0)
    sampler.start()
    sampler.wait_first(5.0)
    res = online.run(windows, per, verify=args.verify, host_windows=200)
    clocks = sampler.stop()
    # what the reference's offline flow would have to do per refresh: rebuild the table over the launches so far
    m = min(CPU_SAMPLE_RECORDS, windows * per)
    rec = trace.generate_fast(trace.config("c5", m), interleave_solo=True)
    t0 = time.perf_counter()
    c_oracle.build_pair_table(rec)
    cpu_ms = 1e3 * (time.perf_counter() - t0)
    line = {
        "metric": "per-window update latency (p50)", "value": res["p50"], "unit": "ms", "n_gpus": 1, "steps": windows - 200, "warmup": 5,
        "ms_per_step": res["mean"], "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "u32/u64 integer, f64 tables",
        "data": "synthetic",
        "config": {"workload": f"c5: resident table, {windows} windows of {per} launches, {res['keys']} keys, {res['pair_rows']} table rows, largest row {res['largest_row_samples']} samples",
                   "l2": "a window is 3 MB: the latency of a short chain of launches, not a bandwidth figure"},
        "p99": res["p99"], "max": res["max"], "p50_by_quarter_of_the_run": res["p50_by_quarter"], "device_ms_p50": res["device_ms_p50"],
        "readout_ms": res["readout_ms"], "verified_against_batch_build": res["verified_against_batch_build"],
        "clocks": clocks, "gpu_launches": int(res["gpu_launches_per_window"] * (windows - 200)),
        "e2e": {"value": res["host_windows"]["p50"], "unit": "ms", "h2d_bytes_per_step": per * RECORD_DTYPE.itemsize, "d2h_bytes_per_step": 128,
                "p99": res["host_windows"]["p99"], "windows": res["host_windows"]["windows"]},
        "roofline": None,
        "cpu_baseline": {"value": cpu_ms, "unit": "ms", "cores": c_oracle.host_threads(), "kind": "port",
                         "sample": f"the reference has no incremental mode: one rebuild of the table over {m} launches with the C/OpenMP oracle, all host threads"},
    }
    print(json.dumps(line), flush=True)


def tenant_runs(dev, n_rec):
    """The same launches as one ordered run per tenant, concatenated: what the agents leave behind, one ordered log per
    process (scheduler/agent.cpp:683-705).  Built on the device from the merged trace (byte 31 of a record is its tenant)."""
    import torch

    rows = dev.view(n_rec, 48)
    tenant = rows[:, 31]
    parts = [rows[tenant == t] for t in torch.unique(tenant).tolist()]
    return torch.cat(parts).reshape(-1).contiguous()


def main():
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.workload.lower() == "c5":
        run_online(args, rank)
        return

    import torch
    import torch.distributed as dist

    from kernel_scheduling_b200 import parallel, trace
    from kernel_scheduling_b200.pair_table import PairTableBuilder
    from kernel_scheduling_b200.records import RECORD_DTYPE

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the GPU arm")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    spec = trace.config(args.workload)
    n_rec = args.records or min(spec.n_records, args.max_records)
    # weak scaling: every rank owns one window of n_rec records of the same workload (same key tables, its own launches);
    # the windows follow one another in time, so the job is ONE trace of world * n_rec records
    spec = trace.config(args.workload, n_rec)
    # one GPU and more records than one call of the ordinary build can take (2^30 overlapping pairs): the streamed build,
    # and the trace is made window by window (the same windows an N-GPU job of this size gives its ranks)
    streamed = world == 1 and (args.streamed or n_rec > 160_000_000)
    gen_window = n_rec if not streamed else min(n_rec, args.gen_window)
    host = torch.empty(gen_window * 48, dtype=torch.uint8).pin_memory()
    rec = host.numpy().view(RECORD_DTYPE)
    t_gen = time.perf_counter()
    if not streamed:
        trace.generate_fast(spec, window=rank, out=rec)
        dev = None
    else:
        dev = torch.empty(n_rec * 48, dtype=torch.uint8, device="cuda")
        shift, done = 0, 0
        while done < n_rec:
            m = min(gen_window, n_rec - done)
            part = trace.generate_fast(trace.config(args.workload, m), window=done // gen_window, out=rec[:m])
            part["start_ns"] += np.uint64(shift)
            part["end_ns"] += np.uint64(shift)
            shift += int(part["start_ns"][-1] - part["start_ns"][0]) + 1
            dev[done * 48: (done + m) * 48].copy_(host[: m * 48])
            done += m
        torch.cuda.synchronize()
    t_gen = time.perf_counter() - t_gen
    if world > 1:
        span = torch.tensor([int(rec["start_ns"][-1] - rec["start_ns"][0]) + 1], dtype=torch.int64, device="cuda")
        spans = [torch.zeros_like(span) for _ in range(world)]
        dist.all_gather(spans, span)
        shift = sum(int(x[0]) for x in spans[:rank])
        rec["start_ns"] += np.uint64(shift)
        rec["end_ns"] += np.uint64(shift)
    first_start = int(rec["start_ns"][0])
    if dev is None:
        dev = host.cuda(non_blocking=False)
    if streamed:
        args.no_e2e = args.no_extras = True  # both need the whole trace in one host buffer
    stream = torch.cuda.Stream()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- the first call on a fresh handle (nothing sized, nothing known about the trace), one GPU only
    extra = {}
    builder = PairTableBuilder(device=local_rank, stream=stream.cuda_stream)
    if world == 1 and not args.no_extras:
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        builder.build_device(dev.data_ptr(), n_rec, time_ordered=True)
        torch.cuda.synchronize()
        extra["first_call_ms"] = {"wall": 1e3 * (time.perf_counter() - t0), "device": builder.info["ms_total"],
                                  "note": "fresh handle: scratch allocation, sample-buffer growth and host read-backs of the counts included"}

    # N > 1: the native driver (exchanges issued by the library through NCCL); --mg-driver python runs the same phases with
    # the exchanges in torch.distributed
    session = parallel.NativeSession(builder, rank, world) if world > 1 and args.mg_driver == "native" else None

    def step_device():
        if streamed:
            return builder.build_streamed_device(dev.data_ptr(), n_rec, window_records=args.window_records, n_parts=args.parts)
        if world == 1:
            return builder.build_device(dev.data_ptr(), n_rec, time_ordered=True)
        if session is not None:
            return session.build_device(dev)
        with torch.cuda.stream(stream):
            keys_t, table_t = parallel.run_distributed(parallel.build_steps(parallel.GpuStages(builder, dev, first_start), rank, world, on_device=True))
        builder.info = {"n_pairs": 0, "n_rows": table_t.numel() // 128, "n_keys": keys_t.numel() // 72}
        return table_t.numel() // 128

    # ---- device-resident: warm-up, then blocks of exactly K timed steps.  The clock sampler (nvidia-smi, rank 0) runs from
    # the warm-up on.  One block is K steps between two CUDA events on the library's stream, bracketed by barriers; blocks
    # are repeated until the timed region is at least MIN_TIMED_S long and the median block is reported.
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        sampler.wait_first(5.0)
    barrier()
    warm = max(args.warmup, 3)
    for _ in range(warm - 1):
        step_device()
    torch.cuda.synchronize()
    t0 = time.perf_counter()  # the last warm-up step alone sizes the timed region (the first ones grow buffers)
    step_device()
    torch.cuda.synchronize()
    est_ms = 1e3 * (time.perf_counter() - t0)
    if args.clock_load_steps > 0 and est_ms * warm < 300.0:  # short steps: more load in front so that the sampler sees steady clocks
        for _ in range(int(min(args.clock_load_steps, 300.0 / max(est_ms, 1e-3)))):
            step_device()
    n_blocks = int(min(50, max(3, -(-1.2 * MIN_TIMED_S * 1e3 // max(est_ms * args.steps, 1e-3))))) if args.clock_load_steps > 0 else 1
    nb = torch.tensor([n_blocks], device="cuda")
    if world > 1:
        dist.all_reduce(nb, op=dist.ReduceOp.MAX)
    n_blocks = int(nb[0])
    stage_names = ("ms_decode", "ms_dict", "ms_join", "ms_sort", "ms_reduce", "ms_finalize", "ms_total")
    stage_ms = {k: 0.0 for k in stage_names}
    launches0 = builder.launch_count
    block_ms = []
    for _ in range(n_blocks):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            for _ in range(args.steps):
                step_device()
                for k in stage_names:
                    stage_ms[k] += builder.info.get(k, 0.0)
            e1.record(stream)
        barrier()
        block_ms.append(e0.elapsed_time(e1))
    clocks = sampler.stop() if rank == 0 else None
    launches = (builder.launch_count - launches0) // n_blocks
    stage_ms = {k: v / n_blocks for k, v in stage_ms.items()}
    info = dict(builder.info)
    phase_ms = None
    whole_rows = None
    if world > 1:
        # device time of the five phases of the sharded build (each with its exchange), as the library measures them when
        # asked to (one more host wait per call, so not inside the timed region)
        if session is not None:
            phase_ms = {}
            for _ in range(3):
                session.build_device(dev, timing=True)
                for k in ("ms_decode", "ms_join", "ms_order", "ms_reduce", "ms_finalize", "ms_total"):
                    phase_ms[k] = phase_ms.get(k, 0.0) + builder.info[k] / 3.0
            whole_rows = int(builder.info["n_rows"])
        stage_ms = {k: 0.0 for k in stage_names}
        # per-kernel times for the roofline: the same kernels over the local window alone, after the timed region
        for i in range(4):  # the first call after the sharded runs has no size hints from a previous call: not counted
            builder.build_device(dev.data_ptr(), n_rec, time_ordered=True)
            for k in stage_names:
                stage_ms[k] += builder.info[k] * args.steps / 3.0 if i else 0.0
        info = dict(builder.info)
        torch.cuda.synchronize()

    # ---- one GPU: the costs the timed steps do not show
    if world == 1 and not args.no_extras:
        def timed(fn, reps=3):
            out = []
            for _ in range(reps):
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                fn()
                torch.cuda.synchronize()
                out.append(1e3 * (time.perf_counter() - t0))
            return statistics.median(out)

        # the same trace without the caller's word for its order: one more host read-back, counts read back between the stages
        extra["unhinted_ms"] = timed(lambda: builder.build_device(dev.data_ptr(), n_rec, time_ordered=False))
        runs = tenant_runs(dev, n_rec)
        builder.build_device(runs.data_ptr(), n_rec, time_ordered=False)
        extra["tenant_runs_ms"] = timed(lambda: builder.build_device(runs.data_ptr(), n_rec, time_ordered=False))
        extra["tenant_runs_note"] = "the same launches as one ordered run per tenant, concatenated: the timeline is sorted by start_ns on the device first"
        rows_runs = int(builder.info["n_rows"])
        del runs
        builder.build_device(dev.data_ptr(), n_rec, time_ordered=True)
        assert rows_runs == int(builder.info["n_rows"]) == int(info["n_rows"])
        if args.verify:
            from oracle import c_oracle
            from tests.helpers import assert_tables_match

            keys_v, pairs_v = builder.fetch()
            assert_tables_match(keys_v, pairs_v, *c_oracle.build_pair_table(rec))
            extra["verified"] = "table equal to the C oracle's on the full trace (exact columns bit for bit, sums and means to 1e-6)"

    # ---- end to end through the public API: host records in, host tables out
    e2e = None
    if not args.no_e2e:
        out_pinned = None

        def step_e2e():
            if world == 1:
                return builder.build(rec, time_ordered=True, pinned=True)
            if session is not None:
                with torch.cuda.stream(stream):
                    dev.copy_(host, non_blocking=True)  # this step's records from pinned host memory
                return session.build(dev, pinned=rank == 0, fetch=rank == 0)  # the whole table back to pinned host memory, on rank 0
            with torch.cuda.stream(stream):
                dev.copy_(host, non_blocking=True)
                keys_t, table_t = parallel.run_distributed(parallel.build_steps(parallel.GpuStages(builder, dev, first_start), rank, world, on_device=True))
                nonlocal out_pinned
                need = keys_t.numel() + table_t.numel()
                if out_pinned is None or out_pinned.numel() < need:
                    out_pinned = torch.empty(need + need // 4, dtype=torch.uint8).pin_memory()
                out_pinned[: keys_t.numel()].copy_(keys_t, non_blocking=True)  # the whole table back to pinned host memory
                out_pinned[keys_t.numel(): need].copy_(table_t, non_blocking=True)
                stream.synchronize()
                return out_pinned[: keys_t.numel()].numpy(), out_pinned[keys_t.numel(): need].numpy()

        for _ in range(2):
            keys, pairs = step_e2e()
        barrier()
        t0 = time.perf_counter()
        e2e_steps = max(1, min(args.steps, 5))
        for _ in range(e2e_steps):
            keys, pairs = step_e2e()
        torch.cuda.synchronize()
        ms_e2e = 1e3 * (time.perf_counter() - t0)
        e2e = {"ms": ms_e2e, "steps": e2e_steps, "h2d": rec.nbytes, "d2h": (keys.nbytes + pairs.nbytes) if keys is not None else 0}

    # ---- max over ranks, block by block
    t = torch.tensor(block_ms + [e2e["ms"] / e2e["steps"] if e2e else 0.0, float(e2e["d2h"]) if e2e else 0.0], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    blocks = sorted(float(x) / args.steps for x in t[:-2])
    ms_e2e_step, d2h = float(t[-2]), int(t[-1])

    if rank == 0:
        total_records = n_rec * world
        ms_per_step = statistics.median(blocks)
        value = total_records / (ms_per_step * 1e-3)
        peaks = {}
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                peaks = json.load(f)
        except OSError:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        peak_src = "measured copy bandwidth (MEASURED_PEAKS.json)" if peaks else "fallback 6650 GB/s"
        per_stage = {k: v / args.steps for k, v in stage_ms.items()}
        P, T, N, S = info.get("n_pairs", 0), info["n_rows"], n_rec, info.get("n_solo", 0)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warm,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u32/u64 integer, f64 tables",
            "data": "synthetic",
            "config": {"workload": workload_label(args.workload),
                       "this_run": f"{n_rec} records per GPU, {info['n_keys']} keys, {P} overlapping pairs per GPU, {T} table rows"
                                   + (f" per window, {whole_rows} in the whole table" if whole_rows else "")
                                   + ("" if world == 1 else f"; one trace of {total_records} records in {world} time windows, samples exchanged by all-to-all, whole table on every rank"),
                       "records_per_gpu": n_rec, "l2": "inputs (48 B x records) larger than L2; no flush needed", "input_order": "start_ns-ordered (verified on device)",
                       **({"build": "streamed: joined window by window, samples kept in key ranges that are sorted and reduced one after the other"} if streamed else {}),
                       "generated_s": round(t_gen, 2)},
            "timed_blocks": {"blocks": len(blocks), "steps_per_block": args.steps, "ms_per_step_min": blocks[0], "ms_per_step_median": ms_per_step,
                             "ms_per_step_max": blocks[-1], "timed_region_s": sum(blocks) * args.steps * 1e-3},
            "clocks": clocks,
            "gpu_launches": int(launches),
            "stage_ms": per_stage,
            **({"phase_ms": phase_ms} if phase_ms else {}),
            **extra,
            "roofline": roofline(per_stage, info, N, S, P, T, ms_per_step, peak, peak_src),
        }
        if e2e:
            line["e2e"] = {"value": total_records / (ms_e2e_step * 1e-3), "unit": UNIT, "h2d_bytes_per_step": int(e2e["h2d"]), "d2h_bytes_per_step": d2h,
                           "ms_per_step": ms_e2e_step}
        if world == 1 and not args.no_cpu_baseline:
            m = min(CPU_SAMPLE_RECORDS, n_rec)
            line["cpu_baseline"] = cpu_baseline(args.workload, m, rec[:m] if m == n_rec and not streamed else None)
        print(json.dumps(line), flush=True)
    if session is not None:
        session.close()  # collective: every rank unmaps the others' buffers before any rank frees its own
    builder.close()
    if world > 1:
        dist.destroy_process_group()


def roofline(per_stage, info, N, S, P, T, ms_per_step, peak, peak_src):
    """The roofline block of the JSON line: the kernel with the largest share of the step, its algorithmic bytes per launch
    over its measured launch time (CUDA events inside the library, on its stream), and the whole path."""
    # algorithmic bytes per launch: decode reads 48 B and writes 16 B per record; the join reads the 16-byte timeline entry
    # of every record and writes a 16-byte sample per pair; one pass of the sample sort reads and writes every 16-byte
    # sample once.  traffic: dram__bytes_read + dram__bytes_write of one ncu capture of the same kernels at 20 M records of
    # c3 (41 M samples: larger than L2, small on the device), per unit, scaled to this run's units -- each of these kernels
    # streams its input once, so its traffic grows in proportion: 63.7 B per record (decode), 16.0 B per record + 14.8 B per
    # pair (join), 31.9 B per sample (a sort pass).
    passes = max(1, int(info.get("sort_passes", 0)) or 1)
    cand = {
        "k_decode_hash": (per_stage["ms_decode"], 64.0 * N, 63.7 * N),
        "k_join": (per_stage["ms_join"], 16.0 * N + 16.0 * P, 16.0 * N + 14.8 * P),
    }
    if info.get("ms_sort_pass", 0.0) > 0.0:
        cand["k_onesweep_pass16"] = (info["ms_sort_pass"], 32.0 * (S + P), 31.9 * (S + P))
    dom = max(cand, key=lambda k: cand[k][0] * (passes if k == "k_onesweep_pass16" else 1))
    ms, alg, traffic = cand[dom]
    achieved = alg / (ms * 1e-3) / 1e9 if ms > 0 else 0.0
    path_bytes = 48.0 * N + 32.0 * P + 96.0 * T
    return {"bound": "hbm", "kernel": dom, "launches_per_step": passes if dom == "k_onesweep_pass16" else 1, "ms_per_launch": ms,
            "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": traffic, "peak_source": peak_src,
            "path_algorithmic_bytes": path_bytes, "path_frac": path_bytes / (ms_per_step * 1e-3) / 1e9 / peak}


if __name__ == "__main__":
    main()
