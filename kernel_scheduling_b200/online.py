"""Online incremental mode (BASELINE config c5): a resident pair table updated window by window.

    python -m kernel_scheduling_b200.online [--windows 200] [--window-records 65536] [--verify]

Feeds a seeded synthetic two-tenant trace (the key and duration distributions of config c2, solo launches interleaved)
to ``PairTableBuilder.update`` in windows of 65,536 launches that arrive in device memory, and prints one JSON line with
the per-window update latency (p50 / p99 / max, host wall clock around the call, which includes its two host waits) and
the device time of an update.  ``--verify`` reads the table out at the end and compares it with a batch build over all
launches (bit for bit except the sums and means, which agree to 1e-6).
"""
from __future__ import annotations

import argparse
import json
import time

import numpy as np


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--windows", type=int, default=200)
    ap.add_argument("--window-records", type=int, default=65536)
    ap.add_argument("--verify", action="store_true")
    args = ap.parse_args(argv)

    import torch

    from . import trace
    from .pair_table import PairTableBuilder

    n = args.windows * args.window_records
    spec = trace.config("c5", n)
    rec = trace.generate(spec, interleave_solo=True)
    dev = torch.from_numpy(rec.view(np.uint8).reshape(-1)).cuda()
    torch.cuda.synchronize()
    wall, device_ms, samples = [], [], 0
    with PairTableBuilder(device=0) as b:
        b.update_begin()
        for w in range(args.windows):
            lo = w * args.window_records
            t0 = time.perf_counter()
            samples += b.update(dev.data_ptr() + lo * 48, args.window_records)
            wall.append(1e3 * (time.perf_counter() - t0))
            device_ms.append(b.update_info["ms_total"])
        t0 = time.perf_counter()
        keys, pairs = b.update_table()
        readout_ms = 1e3 * (time.perf_counter() - t0)
        b.update_end()
        verified = None
        if args.verify:
            bkeys, bpairs = b.build(dev.data_ptr(), n, time_ordered=True)
            ok = keys.tobytes() == bkeys.tobytes() and len(pairs) == len(bpairs)
            for c in bpairs.dtype.names:
                if not ok:
                    break
                if c.startswith(("sum", "mean")):
                    ok = bool(np.allclose(pairs[c], bpairs[c], rtol=1e-6, atol=0, equal_nan=True))
                else:
                    ok = bool(np.array_equal(pairs[c], bpairs[c], equal_nan=True))
            verified = ok
    steady = wall[min(5, len(wall) - 1):]  # the first windows size the buffers
    line = {
        "metric": "per-window update latency", "unit": "ms", "windows": args.windows, "window_records": args.window_records,
        "p50": float(np.percentile(steady, 50)), "p99": float(np.percentile(steady, 99)), "max": float(np.max(steady)),
        "device_ms_p50": float(np.percentile(device_ms[min(5, len(wall) - 1):], 50)),
        "records": n, "samples": int(samples), "keys": int(len(keys)), "pair_rows": int(len(pairs)), "readout_ms": readout_ms,
        "largest_row_samples": int(pairs["count"].max()) if len(pairs) else 0, "verified_against_batch_build": verified,
    }
    print(json.dumps(line), flush=True)
    return 0 if verified in (None, True) else 1


if __name__ == "__main__":
    raise SystemExit(main())
