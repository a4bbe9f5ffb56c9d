"""CPU oracle for the decision-log analytics (pandas).  TEST INFRASTRUCTURE, NOT A PRODUCT PATH.

Restates, with pandas group-bys, what ``kernel_scheduling_b200.decision_log.analyse`` computes on the device from the
daemon's decision log (reference: scheduler/scheduler_daemon.cpp:585-605 for the fields, :674-676 for the header) joined to
the agents' timing logs (scheduler/agent.cpp:692-705) on (pid, kernel_id), as the daemon's own comment prescribes (:587).
The reference ships no analysis of these logs, so this oracle is "parity unpinned": it pins the device path to an
independent restatement, not to reference output.
"""
from __future__ import annotations

import io

import numpy as np
import pandas as pd

WAIT_BINS, BATCH_BINS = 33, 17


def _dims(text):
    import re

    v = [int(x) for x in re.findall(r"\d+", str(text))]
    return tuple(v[:3]) if len(v) >= 3 else None


def analyse(decision_tsv: bytes, agent_tsvs: dict) -> pd.DataFrame:
    """-> one row per (model, kernel_base, block): rows, wait_rows, wait_ns_{sum,min,max,median}, wait_hist, batch_hist,
    dur_{alone,gang}_{rows,median_ns}."""
    d = pd.read_csv(io.BytesIO(decision_tsv), sep="\t", dtype=str, keep_default_na=False)
    d["block_t"] = d["block"].map(_dims)
    d["size"] = pd.to_numeric(d["batch_size"])
    wait = d["queue_wait_us"].map(lambda s: None if s == "" else int(round(float(s) * 1000)))
    d["wait_ns"] = wait
    dur = {}
    for pid, text in agent_tsvs.items():
        a = pd.read_csv(io.BytesIO(text), sep="\t", dtype=str, keep_default_na=False)
        for kid, s, e in zip(a["kernel_id"], a["start_ns"], a["end_ns"]):
            if kid != "" and s != "" and e != "" and int(float(e)) >= int(float(s)):
                dur[(int(pid), int(kid))] = int(float(e)) - int(float(s))
    d["dur"] = [dur.get((int(p), int(k))) if p != "" and k != "" else None for p, k in zip(d["pid"], d["kernel_id"])]
    rows = []
    for (model, base, block), g in d.groupby(["model", "kernel_base", "block_t"], sort=False):
        w = np.array([x for x in g["wait_ns"] if x is not None and x == x], dtype=np.int64)
        w = np.minimum(w, 0xFFFFFFFF)
        whist = np.zeros(WAIT_BINS, np.int64)
        for x in w:
            whist[min(int(x).bit_length(), WAIT_BINS - 1)] += 1
        bhist = np.bincount(np.minimum(g["size"].to_numpy(), BATCH_BINS - 1), minlength=BATCH_BINS)
        row = {"model": model, "kernel": base, "block": block, "rows": len(g), "wait_rows": len(w), "wait_ns_sum": int(w.sum()),
               "wait_ns_min": int(w.min()) if len(w) else 0, "wait_ns_max": int(w.max()) if len(w) else 0,
               "wait_ns_median": float(np.median(w)) if len(w) else float("nan"), "wait_hist": whist, "batch_hist": bhist}
        for tag, sel in (("alone", g["size"] == 1), ("gang", g["size"] >= 2)):
            v = np.array([x for x in g["dur"][sel] if x is not None and x == x], dtype=np.int64)
            row[f"dur_{tag}_rows"] = len(v)
            row[f"dur_{tag}_median_ns"] = float(np.median(np.minimum(v, 0xFFFFFFFF))) if len(v) else float("nan")
        rows.append(row)
    return pd.DataFrame(rows)
