"""Decision-log analytics: queue wait and batch size per kernel, from the daemon's log joined to the agents' logs.

    python -m kernel_scheduling_b200.decision_log <scheduler_<pid>_decisions.tsv> [agent_<pid>_timing.tsv ...] [--out stats.tsv]

The scheduler daemon writes one row per finished kernel (scheduler/scheduler_daemon.cpp:585-605 describes the fields,
:674-676 is the header): the decision that released it (``batch_id``, ``batch_size``, ``batch_pos``), who it was (``pid``,
``kernel_id``, ``kernel_base``, ``grid``, ``block``, ``model``) and how long it waited (``request_ns``, ``post_ns``,
``queue_wait_us``).  The agents' logs (scheduler/agent.cpp:692-705) hold what the kernel then did (``start_ns``,
``end_ns``); the two are joined on (pid, kernel_id), as the daemon's comment says (:587).  The reference ships no analysis of
these logs; this module analyses them with the device-side text parser and the segmented kernels of the pair-table path:

  * both logs are parsed on the device (``ks_tsv_extract``: line splitting, tab walking, integer / decimal / dimension
    fields, 64-bit string hashes),
  * a kernel is (model, kernel_base, block) -- the daemon's TYPE signature (scheduler_daemon.cpp:213) -- hashed to 64 bits,
  * rows are grouped by kernel with the library's radix sort (``ks_sort_pairs_u64``), and per kernel the exact count, sum,
    minimum, maximum and median of the queue wait (``ks_segment_stats``, integer nanoseconds), a log2 histogram of the
    queue wait and a histogram of the batch size (``ks_segment_hist``) come from the segmented kernels,
  * the measured duration of every decision row (agent ``end_ns - start_ns`` of the same (pid, kernel_id)) is reduced the
    same way twice: over the rows released alone (batch_size 1) and over the rows released in a gang.
"""
from __future__ import annotations

import os
import re
import sys

import numpy as np

from . import _lib
from .pair_table import PairTableBuilder

WAIT_BINS = 33   # bit length of the wait in ns: bin b holds waits in [2^(b-1), 2^b)
BATCH_BINS = 17  # batch sizes 0..15, 16 = larger
NONE = np.uint64(0xFFFFFFFFFFFFFFFF)
U32_MAX = 0xFFFFFFFF

DECISION_COLUMNS = [(1, _lib.COL_U64), (5, _lib.COL_U64), (6, _lib.COL_U64), (11, _lib.COL_MILLI), (16, _lib.COL_HASH), (16, _lib.COL_SPAN),
                    (18, _lib.COL_DIMS), (19, _lib.COL_HASH), (19, _lib.COL_SPAN)]
AGENT_COLUMNS = [(0, _lib.COL_U64), (9, _lib.COL_U64), (10, _lib.COL_U64)]


def _mix64(x: np.ndarray) -> np.ndarray:
    x = x.astype(np.uint64).copy()
    with np.errstate(over="ignore"):
        x ^= x >> np.uint64(30)
        x *= np.uint64(0xBF58476D1CE4E5B9)
        x ^= x >> np.uint64(27)
        x *= np.uint64(0x94D049BB133111EB)
        x ^= x >> np.uint64(31)
    return x


def kernel_hash(model_hash, base_hash, block_word) -> np.ndarray:
    """64-bit id of (model, kernel_base, block) from the device's field hashes."""
    with np.errstate(over="ignore"):
        return _mix64(_mix64(np.asarray(model_hash, np.uint64)) ^ _mix64(np.asarray(base_hash, np.uint64) + np.uint64(0x9E3779B97F4A7C15)) ^ np.asarray(block_word, np.uint64))


def _text(path_or_bytes) -> np.ndarray:
    return np.fromfile(path_or_bytes, dtype=np.uint8) if isinstance(path_or_bytes, (str, os.PathLike)) else np.frombuffer(path_or_bytes, dtype=np.uint8)


def _segments(sorted_keys: np.ndarray):
    starts = np.flatnonzero(np.r_[True, sorted_keys[1:] != sorted_keys[:-1]]) if len(sorted_keys) else np.zeros(0, np.int64)
    return starts, np.r_[starts, len(sorted_keys)].astype(np.uint64)


def analyse(decision_log, agent_logs: dict | None = None, builder: PairTableBuilder | None = None) -> dict:
    """decision_log: path or bytes of the daemon's log; agent_logs: {pid: path or bytes of agent_<pid>_timing.tsv}.
    -> dict of columns, one entry per kernel (model, kernel_base, block), ordered by the kernel's 64-bit id:
    model, kernel, block, rows, wait_rows, wait_ns_{sum,min,max,median}, wait_hist [K, 33], batch_hist [K, 17],
    dur_alone_{rows,median_ns}, dur_gang_{rows,median_ns} (NaN medians where no agent row matched)."""
    own = builder is None
    b = builder or PairTableBuilder()
    try:
        text = _text(decision_log)
        size, pid, kid, wait_milli, base_h, base_span, block, model_h, model_span = b.tsv_extract(text, DECISION_COLUMNS)
        n = len(size)
        key = kernel_hash(model_h, base_h, block)
        skey, order = b.sort_pairs(key, np.arange(n, dtype=np.uint64))
        order = order.astype(np.int64)
        starts, offsets = _segments(skey)
        K = len(starts)
        # queue wait in ns (the log prints microseconds with three decimals); rows without one (blank: the request time was
        # not known) are left out of the wait statistics; waits of 2^32 ns (4.3 s) and more are counted as 2^32 - 1
        has_wait = wait_milli[order] != NONE
        worder = order[has_wait]
        wstarts, woff = _segments(skey[has_wait])
        wait_ns = np.minimum(wait_milli[worder], np.uint64(U32_MAX)).astype(np.uint32)
        wstats = b.segment_stats(wait_ns, woff) if len(wstarts) else np.zeros((0, 6), np.uint64)
        whist = b.segment_hist(wait_ns, woff, WAIT_BINS, log2_bins=True) if len(wstarts) else np.zeros((0, WAIT_BINS), np.uint32)
        bsize = np.minimum(size[order], np.uint64(BATCH_BINS - 1)).astype(np.uint32)
        bhist = b.segment_hist(bsize, offsets, BATCH_BINS) if K else np.zeros((0, BATCH_BINS), np.uint32)

        def spread(per_wait_segment, fill, dtype):
            """wait statistics live on the kernels that have at least one wait; put them on all K kernels"""
            out = np.full((K,) + per_wait_segment.shape[1:], fill, dtype=dtype)
            if len(wstarts):
                out[np.searchsorted(skey[starts], skey[has_wait][wstarts])] = per_wait_segment
            return out

        res = {
            "key": skey[starts], "rows": np.diff(offsets.astype(np.int64)).astype(np.uint64),
            "wait_rows": spread(wstats[:, 0], 0, np.uint64), "wait_ns_sum": spread(wstats[:, 1], 0, np.uint64),
            "wait_ns_min": spread(wstats[:, 2], 0, np.uint64), "wait_ns_max": spread(wstats[:, 3], 0, np.uint64),
            "wait_ns_median": spread((wstats[:, 4].astype(np.float64) + wstats[:, 5].astype(np.float64)) * 0.5, np.nan, np.float64),
            "wait_hist": spread(whist, 0, np.uint32), "batch_hist": bhist,
        }
        first = order[starts]  # one row of every kernel, for its strings
        def strings(span):
            return [text[int(s >> np.uint64(20)): int(s >> np.uint64(20)) + int(s & np.uint64((1 << 20) - 1))].tobytes().decode() for s in span[first]]
        res["model"], res["kernel"] = strings(model_span), strings(base_span)
        blk = block[first]
        res["block"] = np.stack([blk & np.uint64(0x1FFFFF), (blk >> np.uint64(21)) & np.uint64(0x1FFFFF), (blk >> np.uint64(42)) & np.uint64(0x1FFFFF)], axis=1).astype(np.uint32)

        # ---- the measured duration of every decision row: the agent's row of the same (pid, kernel_id)
        dur = np.full(n, NONE, dtype=np.uint64)
        for apid, log in (agent_logs or {}).items():
            akid, astart, aend = b.tsv_extract(_text(log), AGENT_COLUMNS)
            ok = (akid != NONE) & (astart != NONE) & (aend != NONE) & (aend >= astart)
            if not ok.any():
                continue
            table = np.full(int(akid[ok].max()) + 1, NONE, dtype=np.uint64)
            table[akid[ok].astype(np.int64)] = aend[ok] - astart[ok]
            mine = (pid == np.uint64(apid)) & (kid != NONE) & (kid < np.uint64(len(table)))
            dur[mine] = table[kid[mine].astype(np.int64)]
        for tag, cls in (("alone", size[order] == 1), ("gang", (size[order] >= 2) & (size[order] != NONE))):
            sel = cls & (dur[order] != NONE)
            dstarts, doff = _segments(skey[sel])
            d = np.minimum(dur[order][sel], np.uint64(U32_MAX)).astype(np.uint32)
            st = b.segment_stats(d, doff) if len(dstarts) else np.zeros((0, 6), np.uint64)
            rows, med = np.zeros(K, np.uint64), np.full(K, np.nan)
            if len(dstarts):
                at = np.searchsorted(skey[starts], skey[sel][dstarts])
                rows[at] = st[:, 0]
                med[at] = (st[:, 4].astype(np.float64) + st[:, 5].astype(np.float64)) * 0.5
            res[f"dur_{tag}_rows"], res[f"dur_{tag}_median_ns"] = rows, med
        return res
    finally:
        if own:
            b.close()


def write_tsv(res: dict, path) -> None:
    with open(path, "w") as f:
        f.write("model\tkernel\tblock\trows\twait_rows\twait_us_median\twait_us_mean\twait_us_max\tbatch_size_mean\tdur_alone_us_median\tdur_gang_us_median\t"
                + "\t".join(f"wait_lt_2^{b}_ns" for b in range(WAIT_BINS)) + "\t" + "\t".join(f"batch_{s}" for s in range(BATCH_BINS)) + "\n")
        for i in range(len(res["key"])):
            wr = int(res["wait_rows"][i])
            bh = res["batch_hist"][i].astype(np.float64)
            cells = [res["model"][i], res["kernel"][i], "(%d, %d, %d)" % tuple(res["block"][i]), str(int(res["rows"][i])), str(wr),
                     f"{res['wait_ns_median'][i] / 1e3:.3f}", f"{(res['wait_ns_sum'][i] / wr / 1e3) if wr else float('nan'):.3f}", f"{res['wait_ns_max'][i] / 1e3:.3f}",
                     f"{(bh * np.arange(BATCH_BINS)).sum() / max(bh.sum(), 1):.3f}", f"{res['dur_alone_median_ns'][i] / 1e3:.3f}", f"{res['dur_gang_median_ns'][i] / 1e3:.3f}"]
            cells += [str(int(v)) for v in res["wait_hist"][i]] + [str(int(v)) for v in res["batch_hist"][i]]
            f.write("\t".join(cells) + "\n")


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    out = None
    if "--out" in argv:
        i = argv.index("--out")
        out = argv[i + 1]
        del argv[i: i + 2]
    if not argv:
        print(__doc__, file=sys.stderr)
        return 2
    agents = {}
    for p in argv[1:]:
        m = re.search(r"agent_(\d+)_timing", os.path.basename(p))
        if not m:
            print(f"{p}: cannot tell the pid from the file name (agent_<pid>_timing.tsv)", file=sys.stderr)
            return 2
        agents[int(m.group(1))] = p
    res = analyse(argv[0], agents)
    if out:
        write_tsv(res, out)
    print(f"{len(res['key'])} kernels, {int(res['rows'].sum())} decision rows, {int(res['wait_rows'].sum())} with a queue wait, "
          f"{int(res['dur_alone_rows'].sum() + res['dur_gang_rows'].sum())} joined to an agent row")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
