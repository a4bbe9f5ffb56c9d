"""The pooling step of the reference's ``profiling/ncu-bench/ncu_summary.py`` on the GPU.

    python -m kernel_scheduling_b200.ncu_summary <launches.csv> <summary.csv>

The reference script walks Nsight Compute reports, turns every profiled launch into one value per label
(ncu_summary.py:196-218) and then pools the launches of each (kernel name, block) group into a mean and a sample
standard deviation per label (:232-241), which is the CSV ``profile_postprocess.combine_duplicates`` reads.  Here the
per-launch values arrive as a frame (or a CSV) with the columns ``Kernel, Block, <label> ...`` -- an empty cell where a
launch has no such metric -- and ``pool_launches`` returns the reference's summary frame: ``Kernel, Block, Launches`` and
``<label>, <label> std`` per label, groups ordered by (name, block) (:233).  The grouping (a stable radix sort of the
rows by group id) and the two-pass reduction run on the device (``ks_pool_launches``).

``per_launch_labels`` restates the two derived labels (:205-211): blocks per wave and duration per wave.
"""
from __future__ import annotations

import math
import sys

import numpy as np
import pandas as pd

from .pair_table import PairTableBuilder

RATIO_LABEL = "Duration/Wave (us)"  # ncu_summary.py:55
BPW_LABEL = "Blocks/Wave"           # :56


def per_launch_labels(duration_us, waves, grid_total):
    """-> (blocks per wave, duration per wave) of launches; NaN where an input is missing or not finite (:205-211)."""
    dur = np.asarray(duration_us, dtype=np.float64)
    w = np.asarray(waves, dtype=np.float64)
    g = np.asarray(grid_total, dtype=np.float64)
    ok_w = np.isfinite(w) & (w > 0)
    with np.errstate(divide="ignore", invalid="ignore"):
        bpw = np.where(ok_w & np.isfinite(g), g / w, np.nan)
        whole = np.maximum(1.0, np.ceil(w - 1e-6))
        ratio = np.where(ok_w & np.isfinite(dur), dur / whole, np.nan)
    return bpw, ratio


def _block_order(block: str):
    """The reference sorts groups by (name, block dims or ()) (:233); its CSV spells the dims '(x, y, z)' or 'n total' (:150-156)."""
    nums = [int(v) for v in "".join(ch if ch.isdigit() else " " for ch in str(block)).split()]
    return tuple(nums)


def pool_launches(df: pd.DataFrame, builder: PairTableBuilder | None = None) -> pd.DataFrame:
    keys = ["Kernel", "Block"]
    labels = [c for c in df.columns if c not in keys]
    pairs = list(dict.fromkeys(zip(df["Kernel"].astype(str), df["Block"].astype(str))))
    pairs.sort(key=lambda kb: (kb[0], _block_order(kb[1]) if kb[1] != "n/a" else ()))
    index = {kb: i for i, kb in enumerate(pairs)}
    gid = np.fromiter((index[kb] for kb in zip(df["Kernel"].astype(str), df["Block"].astype(str))), dtype=np.uint32, count=len(df))
    values = df[labels].apply(pd.to_numeric, errors="coerce").to_numpy(dtype=np.float64)
    own = builder is None
    b = builder or PairTableBuilder()
    try:
        launches, mean, std = b.pool_launches(gid, values, len(pairs))
    finally:
        if own:
            b.close()
    out = pd.DataFrame({"Kernel": [kb[0] for kb in pairs], "Block": [kb[1] for kb in pairs], "Launches": launches.astype(np.int64)})
    for j, label in enumerate(labels):
        out[label] = mean[:, j]
        out[f"{label} std"] = std[:, j]
    return out


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if len(argv) != 2:
        print(__doc__, file=sys.stderr)
        return 2
    pool_launches(pd.read_csv(argv[0], float_precision="round_trip")).to_csv(argv[1], index=False)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
