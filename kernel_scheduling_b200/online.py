"""Online incremental mode (benchmark configuration c5): a resident pair table updated window by window.

    python -m kernel_scheduling_b200.online [--windows 10000] [--window-records 65536] [--verify] [--publish-every K]

Feeds a seeded synthetic two-tenant trace (the key and duration distributions of config c2, solo launches interleaved)
to ``PairTableBuilder.update`` in windows of 65,536 launches that arrive in device memory, and prints one JSON line with
the per-window update latency (p50 / p99 / max, host wall clock around the call, which includes its two host waits) and
the device time of an update.  The trace is generated in stretches of a few hundred windows on the host's cores while
the GPU works on the stretch before, so the run is as long as the configuration asks for (10,000 windows, 655 M launches)
without holding more than two stretches in host memory.

``--verify`` keeps every launch in device memory (48 bytes each: 31 GB for the full run), reads the table out at the end
and compares it with a batch build over all launches (bit for bit except the sums and means, which agree to 1e-6).
``--publish-every K`` reads the table out every K windows and publishes it in the shared-memory segment a scheduler maps
(``pair_table_shm``; the reference's daemon keeps its table in a map filled once at start, scheduler_daemon.cpp:230-274).
"""
from __future__ import annotations

import argparse
import json
import threading
import time

import numpy as np

STRETCH_WINDOWS = 250  # windows generated at a time


def stretches(windows: int, per: int, workload: str = "c5"):
    """Yields (first_window, records) for stretches of the online trace: stretch s is an independent piece of the same
    workload (same key tables, its own launches) shifted in time behind stretch s - 1.  The next stretch is generated on a
    thread of its own while the caller works on the current one."""
    from . import trace

    t0_ns = trace.config(workload).t0_ns

    def make(s, count, shift):
        rec = trace.generate_fast(trace.config(workload, count * per), window=s, interleave_solo=True)
        rec["start_ns"] += np.uint64(shift)
        rec["end_ns"] += np.uint64(shift)
        return rec

    plan = [(s, w, min(STRETCH_WINDOWS, windows - w)) for s, w in enumerate(range(0, windows, STRETCH_WINDOWS))]
    box = {}
    cur = make(plan[0][0], plan[0][2], 0) if plan else None
    for i, (s, first, count) in enumerate(plan):
        th = None
        if i + 1 < len(plan):
            # the next stretch begins behind the last end of this one (launches of a stretch never reach into the next)
            nxt = plan[i + 1]
            shift = int(cur["end_ns"].max()) + 1 - t0_ns
            th = threading.Thread(target=lambda: box.__setitem__(nxt[0], make(nxt[0], nxt[2], shift)))
            th.start()
        yield first, cur
        if th is not None:
            th.join()
            cur = box.pop(plan[i + 1][0])


def run(windows: int = 10_000, per: int = 65_536, verify: bool = False, publish_every: int = 0, host_windows: int = 0, shm_name: str | None = None):
    """Runs the online configuration; returns the result dict (latencies in ms).  ``host_windows``: that many windows at the
    end arrive in pinned HOST memory instead (their copy to the device is part of the update)."""
    import torch

    from . import pair_table_shm
    from .pair_table import PairTableBuilder

    wall, device_ms, host_wall, samples, records = [], [], [], 0, 0
    publish_ms = []
    keep = torch.empty(windows * per * 48, dtype=torch.uint8, device="cuda") if verify else None
    readout_ms, verified, launches = 0.0, None, 0
    with PairTableBuilder(device=0) as b:
        b.update_begin()
        pinned = b.pinned_records(per) if host_windows else None
        l0 = b.launch_count
        for first, rec in stretches(windows, per):
            n_w = len(rec) // per
            if keep is not None:
                dev = keep[first * per * 48: (first + n_w) * per * 48]
                dev.copy_(torch.from_numpy(rec.view(np.uint8).reshape(-1)))
            else:
                dev = torch.from_numpy(rec.view(np.uint8).reshape(-1)).cuda()
            torch.cuda.synchronize()
            for w in range(n_w):
                g = first + w
                if g >= windows - host_windows:
                    pinned[:] = rec[w * per: (w + 1) * per]
                    t0 = time.perf_counter()
                    samples += b.update(pinned)
                    host_wall.append(1e3 * (time.perf_counter() - t0))
                else:
                    t0 = time.perf_counter()
                    samples += b.update(dev.data_ptr() + w * per * 48, per)
                    wall.append(1e3 * (time.perf_counter() - t0))
                    device_ms.append(b.update_info["ms_total"])
                records += per
                if publish_every and (g + 1) % publish_every == 0:
                    t0 = time.perf_counter()
                    keys, pairs = b.update_table()
                    names = [f"kernel_{i}" for i in range(int(keys["name_id"].max()) + 1)] if len(keys) else []
                    models = [f"model_{i}" for i in range(int(keys["tenant"].max()) + 1)] if len(keys) else []
                    empty = (keys[:0], pairs[:0])
                    pair_table_shm.publish((keys, pairs), empty, names, models, name=shm_name or pair_table_shm.SHM_NAME, generation=g + 1)
                    publish_ms.append(1e3 * (time.perf_counter() - t0))
        launches = b.launch_count - l0
        t0 = time.perf_counter()
        keys, pairs = b.update_table()
        readout_ms = 1e3 * (time.perf_counter() - t0)
        b.update_end()
        if verify:
            bkeys, bpairs = b.build(keep.data_ptr(), windows * per, time_ordered=True)
            ok = keys.tobytes() == bkeys.tobytes() and len(pairs) == len(bpairs)
            for c in bpairs.dtype.names:
                if not ok:
                    break
                if c.startswith(("sum", "mean")):
                    ok = bool(np.allclose(pairs[c], bpairs[c], rtol=1e-6, atol=0, equal_nan=True))
                else:
                    ok = bool(np.array_equal(pairs[c], bpairs[c], equal_nan=True))
            verified = ok
    steady = wall[min(5, max(len(wall) - 1, 0)):]  # the first windows size the buffers
    res = {
        "metric": "per-window update latency", "unit": "ms", "windows": windows, "window_records": per,
        "p50": float(np.percentile(steady, 50)), "p99": float(np.percentile(steady, 99)), "max": float(np.max(steady)), "mean": float(np.mean(steady)),
        "device_ms_p50": float(np.percentile(device_ms[min(5, max(len(wall) - 1, 0)):], 50)),
        "p50_by_quarter": [float(np.percentile(q, 50)) for q in np.array_split(np.array(steady), 4)],
        "records": records, "samples": int(samples), "keys": int(len(keys)), "pair_rows": int(len(pairs)), "readout_ms": readout_ms,
        "largest_row_samples": int(pairs["count"].max()) if len(pairs) else 0, "verified_against_batch_build": verified,
        "gpu_launches_per_window": launches / max(windows, 1),
    }
    if host_wall:
        res["host_windows"] = {"windows": len(host_wall), "p50": float(np.percentile(host_wall, 50)), "p99": float(np.percentile(host_wall, 99))}
    if publish_ms:
        res["publish"] = {"every": publish_every, "times": len(publish_ms), "ms_p50": float(np.percentile(publish_ms, 50)), "ms_max": float(np.max(publish_ms)),
                          "note": "read-out of the whole table + shared-memory image (tmp + rename)"}
    return res


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--windows", type=int, default=10_000)
    ap.add_argument("--window-records", type=int, default=65536)
    ap.add_argument("--verify", action="store_true")
    ap.add_argument("--publish-every", type=int, default=0)
    args = ap.parse_args(argv)
    res = run(args.windows, args.window_records, args.verify, args.publish_every, shm_name="/kernel_sched_pairtab_online" if args.publish_every else None)
    if args.publish_every:
        from . import pair_table_shm

        pair_table_shm.unlink("/kernel_sched_pairtab_online")
    print(json.dumps(res), flush=True)
    return 0 if res["verified_against_batch_build"] in (None, True) else 1


if __name__ == "__main__":
    raise SystemExit(main())
