"""Drop-in for the reference's ``postprocess/profile_postprocess.py``.

    python -m kernel_scheduling_b200.profile_postprocess <in.csv> <out.csv>

``combine_duplicates(df)`` keeps the reference's signature and output frame (profile_postprocess.py:5-27): rows
of an NCU summary CSV are grouped by (Kernel, Block); every value column becomes the Launches-weighted mean over
the rows whose cell is not NaN (an all-NaN group stays NaN, the ``min_count=1`` of :14 and :21), ``Launches``
becomes the group total (:25); ``Grid`` and the ``Shared Mem Pipe %`` columns are dropped (:7).  The grouping
(stable radix sort of the rows by group) and the weighted reduction run on the GPU (``ks_combine_duplicates``).
"""
from __future__ import annotations

import sys

import numpy as np
import pandas as pd

from .pair_table import PairTableBuilder


def combine_duplicates(df: pd.DataFrame, builder: PairTableBuilder | None = None) -> pd.DataFrame:
    keys = ["Kernel", "Block"]
    cols_to_excl = ["Launches", "Grid", "Shared Mem Pipe %", "Shared Mem Pipe % std"] + keys
    value_cols = [c for c in df.columns if c not in cols_to_excl]
    # dense group ids in the order pandas' groupby emits groups (sorted by key)
    group_index = pd.MultiIndex.from_frame(df[keys])
    uniq = group_index.unique().sort_values()
    gid = uniq.get_indexer(group_index).astype(np.uint32)
    own = builder is None
    b = builder or PairTableBuilder()
    try:
        total, means = b.combine_duplicates(gid, df["Launches"].to_numpy(dtype=np.float64), df[value_cols].to_numpy(dtype=np.float64), len(uniq))
    finally:
        if own:
            b.close()
    out = uniq.to_frame(index=False)
    launches = df["Launches"]
    out["Launches"] = total.astype(launches.dtype) if np.issubdtype(launches.dtype, np.integer) else total
    for j, c in enumerate(value_cols):
        out[c] = means[:, j]
    return out


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if len(argv) != 2:
        print(__doc__, file=sys.stderr)
        return 2
    combine_duplicates(pd.read_csv(argv[0])).to_csv(argv[1], index=False)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
