"""Agent timing logs in, ``pair_eff.tsv`` / ``kernel_us.tsv`` out -- the program the reference's daemon names as
``make_pair_eff.py`` (scheduler/scheduler_daemon.cpp:5, :193, :848) but does not ship.

    python -m kernel_scheduling_b200.make_pair_eff --corun a.tsv b.tsv [...] --solo sa.tsv sb.tsv [...] --out-dir DIR
    python -m kernel_scheduling_b200.make_pair_eff --corun agent_<pid>_timing.tsv [...] --pairprof-log pairprof_log_<pid>.tsv --out-dir DIR

Input: the 17-column logs the agent writes (scheduler/agent.cpp:692-705), one file per process; ``--solo`` files
come from a one-kernel-at-a-time run (profiling/pairprof_daemon.cpp:46).  Rows without ``end_ns`` (no completion
callback, agent.cpp:702) are dropped.  With ``--pairprof-log`` (the profiling daemon's own log of the run,
pairprof_daemon.cpp:266, :317-318) every launch is labelled by it instead: kind ``alone*`` = a solo sample, ``gang*`` =
a co-run launch, not mentioned (warm-up) = dropped; the process id comes from the agent log's file name.  The logs are parsed on the GPU (``records_from_log``); ``TraceIngest.records``
is the same ingest from a pandas frame.  Kernel symbols are reduced to their short names (kernel_key.hpp) and
numbered; the ``model`` column is the tenant.

Output, in the layout ``load_pair_eff`` / ``load_kernel_us`` parse (scheduler_daemon.cpp:193-202, :230-264):
SHAPE rows (with grid) and TYPE rows (grid ``*``) in the same files; ``gangs`` = how often the pair overlapped;
extra statistic columns are appended after the ones the daemon reads (it finds columns by name and ignores others).
"""
from __future__ import annotations

import argparse
import os
import re

import numpy as np
import pandas as pd

from . import _lib
from .pair_table import PairTableBuilder
from .records import RECORD_DTYPE, pack_records

_DIMS = re.compile(r"\d+")


def _dims(col: pd.Series) -> np.ndarray:
    """'(x, y, z)' or 'x,y,z' -> (n, 3) uint32 (scheduler_daemon.cpp:214-219 accepts both spellings)."""
    uniq = {s: [int(v) for v in _DIMS.findall(str(s))][:3] for s in col.unique()}
    bad = [s for s, v in uniq.items() if len(v) != 3]
    if bad:
        raise ValueError(f"not a dimension triple: {bad[0]!r}")
    return np.array([uniq[s] for s in col], dtype=np.uint32).reshape(len(col), 3)


class TraceIngest:
    """Turns timing frames into launch records, numbering kernel names and models as it goes."""

    def __init__(self):
        self.names: list[str] = []
        self._name_id: dict[str, int] = {}
        self._base_cache: dict[str, str] = {}
        self.models: list[str] = []

    def name_id(self, symbol: str) -> int:
        """Id of the symbol's canonical short name (new names are numbered in order of appearance)."""
        base = self._base_cache.get(symbol)
        if base is None:
            base = self._base_cache[symbol] = _lib.function_base(str(symbol))
        if base not in self._name_id:
            self._name_id[base] = len(self.names)
            self.names.append(base)
        return self._name_id[base]

    def tenant_id(self, model: str) -> int:
        if model not in self.models:
            self.models.append(model)
        return self.models.index(model)

    def _name_ids(self, symbols: pd.Series) -> np.ndarray:
        ids = {sym: self.name_id(sym) for sym in symbols.unique()}
        return symbols.map(ids).to_numpy(dtype=np.uint32)

    def records(self, frame: pd.DataFrame, solo: bool, pairprof: pd.DataFrame | None = None, pid: int | None = None) -> np.ndarray:
        """``pairprof`` (the profiling daemon's log as a frame) with ``pid``: the solo flag is per launch, from the log's
        ``kind`` of (pid, kernel_id); launches the log does not mention are dropped.  Names and models are numbered over
        all launches with an ``end_ns``, dropped or not (as the device route does)."""
        f = frame[frame["end_ns"].notna()]
        tenants = np.array([self.tenant_id(m) for m in f["model"].astype(str)], dtype=np.uint32)
        name_ids = self._name_ids(f["kernel_name"])
        solo_col = np.full(len(f), solo)
        keep = np.ones(len(f), dtype=bool)
        if pairprof is not None:
            mine = pairprof[pairprof["pid"] == pid]
            kind = dict(zip(mine["kernel_id"].astype(np.int64), mine["kind"].astype(str)))
            kinds = [kind.get(int(k), "") for k in f["kernel_id"]]
            keep = np.array([k.startswith(("alone", "gang")) for k in kinds], dtype=bool)
            solo_col = np.array([k.startswith("alone") for k in kinds], dtype=bool)
        f = f[keep]
        n = len(f)
        return pack_records(
            name_ids[keep], _dims(f["grid"]), _dims(f["block"]), np.zeros(n, np.uint32), tenants[keep],
            solo_col[keep], f["start_ns"].to_numpy(dtype=np.uint64), f["end_ns"].to_numpy(dtype=np.uint64))


def agent_pid(path) -> int | None:
    """The process id in an agent log's file name (``agent_<pid>_timing.tsv``, scheduler/agent.cpp:692), or None."""
    m = re.search(r"agent_(\d+)_timing", os.path.basename(str(path)))
    return int(m.group(1)) if m else None


def _text_of(path_or_bytes) -> np.ndarray:
    return np.fromfile(path_or_bytes, dtype=np.uint8) if isinstance(path_or_bytes, (str, os.PathLike)) else np.frombuffer(path_or_bytes, dtype=np.uint8)


def records_from_log(ing: "TraceIngest", builder: PairTableBuilder, path_or_bytes, solo: bool, pairprof_log=None, pid: int | None = None) -> np.ndarray:
    """One agent timing log -> launch records, parsed on the GPU (``ks_tsv_parse``): line splitting, tab walking, number
    and dimension parsing and the string dictionaries run on the device; the host only canonicalises each DISTINCT kernel
    symbol (``ks_function_base``) and numbers names and models in their order of first appearance -- the same ids the
    pandas route (``TraceIngest.records``) assigns.  ``pairprof_log`` (path or bytes of the profiling daemon's log) with
    ``pid``: that log, parsed on the device too (``ks_tsv_label``), decides per launch between solo sample, co-run launch
    and dropped."""
    text = _text_of(path_or_bytes)
    lib, h = builder._lib, builder._h
    n = builder._check(lib.ks_tsv_parse(h, _lib.ptr(text), len(text), 0), "ks_tsv_parse")
    if pairprof_log is not None:
        if pid is None:
            raise ValueError("pid is required with a pairprof log")
        log = _text_of(pairprof_log)
        n = builder._check(lib.ks_tsv_label(h, _lib.ptr(log), len(log), int(pid), 0), "ks_tsv_label")
    maps = []
    for which, slots in ((0, 65536), (1, 256)):
        hashes, where = np.zeros(slots, dtype=np.uint64), np.zeros(slots, dtype=np.uint64)
        builder._check(lib.ks_tsv_dictionary(h, which, _lib.ptr(hashes), _lib.ptr(where)), "ks_tsv_dictionary")
        used = np.flatnonzero(hashes)
        used = used[np.argsort(where[used] >> np.uint64(20), kind="stable")]  # order of first appearance in the file
        ids = np.zeros(slots, dtype=np.uint32)
        for slot in used:
            off, ln = int(where[slot] >> np.uint64(20)), int(where[slot] & np.uint64((1 << 20) - 1))
            string = text[off: off + ln].tobytes().decode()
            ids[slot] = ing.name_id(string) if which == 0 else ing.tenant_id(string)
        maps.append(ids)
    rec = np.zeros(n, dtype=RECORD_DTYPE)
    builder._check(lib.ks_tsv_finish(h, _lib.ptr(maps[0]), _lib.ptr(maps[1]), int(bool(solo)), _lib.ptr(rec), n, 0), "ks_tsv_finish")
    return rec


def _xyz(v) -> str:
    return f"{int(v[0])},{int(v[1])},{int(v[2])}"


def write_tables(out_dir, tables, names, models):
    """tables: [(key_rows, pair_rows, is_type)]. Writes kernel_us.tsv and pair_eff.tsv into out_dir."""
    os.makedirs(out_dir, exist_ok=True)
    us_path, eff_path = os.path.join(out_dir, "kernel_us.tsv"), os.path.join(out_dir, "pair_eff.tsv")
    with open(us_path, "w") as fu, open(eff_path, "w") as fe:
        fu.write("model\tkernel\tblock\tgrid\tsolo_us\tlaunches\tsolo_launches\n")
        fe.write("model_a\tkernel_a\tblock_a\tgrid_a\tmodel_b\tkernel_b\tblock_b\tgrid_b\tefficiency\tgangs"
                 "\tslowdown_median_a\tslowdown_mean_a\tslowdown_min_a\tslowdown_max_a\tslowdown_median_b\tslowdown_mean_b\tslowdown_min_b\tslowdown_max_b\n")
        for keys, pairs, is_type in tables:
            ident = {}
            for r in keys:
                grid = "*" if is_type else _xyz(r["grid"])
                ident[int(r["key"])] = (models[int(r["tenant"])], names[int(r["name_id"])], _xyz(r["block"]), grid)
                if np.isfinite(r["solo_ns"]):
                    fu.write("\t".join(ident[int(r["key"])]) + f"\t{float(r['solo_ns']) / 1e3!r}\t{int(r['launches'])}\t{int(r['solo_launches'])}\n")
            for p in pairs:
                if not np.isfinite(p["efficiency"]):
                    continue  # a pair without both solo times has no efficiency: the daemon would skip the row anyway
                stats = "\t".join(repr(float(p[c])) for c in ("median_a", "mean_a", "min_a", "max_a", "median_b", "mean_b", "min_b", "max_b"))
                fe.write("\t".join(ident[int(p["key_a"])]) + "\t" + "\t".join(ident[int(p["key_b"])]) + f"\t{float(p['efficiency'])!r}\t{int(p['count'])}\t{stats}\n")
    return us_path, eff_path


def build_tables(records: np.ndarray, builder: PairTableBuilder | None = None):
    """-> [(key_rows, pair_rows, is_type)] for the SHAPE keys and the TYPE keys."""
    own = builder is None
    b = builder or PairTableBuilder()
    try:
        return [(*b.build(records, key_type=t), t) for t in (False, True)]
    finally:
        if own:
            b.close()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--corun", nargs="+", required=True)
    ap.add_argument("--solo", nargs="*", default=[])
    ap.add_argument("--pairprof-log", default=None, help="pairprof_log_<pid>.tsv of the run that wrote the --corun logs: labels every launch")
    ap.add_argument("--out-dir", default=".")
    ap.add_argument("--publish-shm", default=None, metavar="NAME",
                    help="also publish both tables as a shared-memory segment (e.g. /kernel_sched_pairtab_v1; include/ks_pairtab_shm.h reads it)")
    args = ap.parse_args(argv)
    ing = TraceIngest()
    with PairTableBuilder() as b:
        if args.pairprof_log:
            pids = [agent_pid(p) for p in args.corun]
            if None in pids:
                ap.error("--pairprof-log needs agent logs named agent_<pid>_timing.tsv")
            parts = [records_from_log(ing, b, p, solo=False, pairprof_log=args.pairprof_log, pid=pid) for p, pid in zip(args.corun, pids)]
        else:
            parts = [records_from_log(ing, b, p, solo=False) for p in args.corun]
        parts += [records_from_log(ing, b, p, solo=True) for p in args.solo]
        rec = np.concatenate(parts)
        tables = build_tables(rec, b)
        us, eff = write_tables(args.out_dir, tables, ing.names, ing.models)
        if args.publish_shm:
            from . import pair_table_shm

            by_type = {is_type: (keys, pairs) for keys, pairs, is_type in tables}
            nbytes = pair_table_shm.publish(by_type[False], by_type[True], ing.names, ing.models, name=args.publish_shm)
            print(f"published {nbytes} bytes as {args.publish_shm}")
    print(f"{len(rec)} launches, {len(ing.names)} kernel names, {len(ing.models)} models -> {us}, {eff}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
