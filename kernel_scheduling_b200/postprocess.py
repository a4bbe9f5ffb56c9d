"""Drop-in for the reference's ``scheduler/postprocess.py``: same command line, same printed lines.

    python -m kernel_scheduling_b200.postprocess <timing_tsv_1> <timing_tsv_2> [--no-progress]

The reference reads two agent timing logs (scheduler/postprocess.py:12-13; the first cut to its last 200,000
rows), prints their lengths (:15), then for every distinct ``start_ns`` prints a running index (:20, :32) and
counts whether one or two launches share that timestamp, and finally prints ``[n_alone, n_pairs]`` (:41).
Here the two files are parsed on the GPU (``ks_tsv_extract``: line splitting and the ``start_ns`` column) and the two
columns stay there for the count (``ks_count_batches``: two radix sorts and one intersection kernel); a duplicate timestamp inside a file raises AssertionError exactly where the reference's ``assert``
would (:24, :36).  ``--no-progress`` drops the index lines, which only exist to show the quadratic loop is alive.
"""
from __future__ import annotations

import sys

import numpy as np

from . import _lib
from .pair_table import PairTableBuilder


def count_batches(start1, start2, builder: PairTableBuilder | None = None):
    """[n_alone, n_pairs] for two arrays of start_ns (file 1 already cut to its last 200,000 rows)."""
    own = builder is None
    b = builder or PairTableBuilder()
    try:
        return b.count_batches(np.asarray(start1, dtype=np.uint64), np.asarray(start2, dtype=np.uint64))
    except _lib.KsError as e:
        if e.status == _lib.ERR_DUPLICATE:
            raise AssertionError("a start_ns occurs more than once in one file") from e
        raise
    finally:
        if own:
            b.close()


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    progress = "--no-progress" not in argv
    files = [a for a in argv if not a.startswith("--")]
    if len(files) != 2:
        print(__doc__, file=sys.stderr)
        return 2
    with PairTableBuilder() as b:
        # the start_ns column of both files (found by its name in the header line, as pandas does), parsed on the device
        cols = []
        for f in files:
            text = np.fromfile(f, dtype=np.uint8)
            header = bytes(text[: 4096]).split(b"\n", 1)[0].rstrip(b"\r").split(b"\t")
            cols.append(b.tsv_extract(text, [(header.index(b"start_ns"), _lib.COL_U64)])[0])
        s1, s2 = cols
        s1 = s1[-200000:]
        print(len(s1), len(s2))
        result = count_batches(s1, s2, b)
    if progress:
        out = sys.stdout
        for n in (len(np.unique(s1)), len(np.unique(s2))):
            out.write("".join(f"{i}\n" for i in range(n)))
    print(result)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
