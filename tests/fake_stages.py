"""A numpy stand-in for one rank's compute (parallel.GpuStages) so that the multi-rank logic -- halos, pair ownership,
global key ids, splitters, the sample exchange, the merges -- can be exercised on the CPU (in one process or as gloo ranks)
and compared with the single-process oracle.  Test infrastructure only."""
import numpy as np
import torch

from kernel_scheduling_b200.parallel import HIST_BINS
from kernel_scheduling_b200.records import KEY_ROW_DTYPE, PAIR_ROW_DTYPE, RECORD_DTYPE
from oracle import pair_table_oracle as O

SOLO = np.uint32(1 << 23)


class FakeStages:
    def __init__(self, records: np.ndarray):
        self.own = np.ascontiguousarray(records, dtype=RECORD_DTYPE)
        self.device = torch.device("cpu")
        self.halo_rec = np.zeros(0, dtype=RECORD_DTYPE)

    def zeros(self, shape, dtype):
        return torch.zeros(shape, dtype=dtype)

    def tensor(self, data, dtype):
        return torch.tensor(data, dtype=dtype)

    def from_bytes(self, raw):
        return torch.frombuffer(bytearray(raw), dtype=torch.uint8) if raw else torch.zeros(0, dtype=torch.uint8)

    def first_start(self):
        return int(self.own["start_ns"][0]) if len(self.own) else None

    def begin(self, key_type):
        self.mode = O.KEY_TYPE if key_type else O.KEY_SHAPE

    def tail(self):
        r = self.own
        if not len(r):
            return torch.zeros(0, dtype=torch.uint8)
        last = r["start_ns"][-1]
        t = r[((r["smem_word"] & SOLO) == 0) & (r["end_ns"] > last)]
        return self.from_bytes(t.tobytes())

    def halo(self, t):
        self.halo_rec = np.frombuffer(t.numpy().tobytes(), dtype=RECORD_DTYPE)

    def _words(self, rec):
        w = np.zeros((len(rec), 8), dtype=np.uint32)
        w[:, 0] = rec["name_id"]
        w[:, 4:7] = rec["block"]
        if self.mode == O.KEY_SHAPE:
            w[:, 1:4] = rec["grid"]
            w[:, 7] = rec["smem_word"] & ~SOLO
        else:
            w[:, 7] = rec["smem_word"] & np.uint32(0xFF000000)
        return w

    def local_keys(self):
        allrec = np.concatenate([self.halo_rec, self.own])
        keys = O.kernel_keys(allrec, self.mode)
        u, first = np.unique(keys, return_index=True)
        words = self._words(allrec[first])
        return torch.from_numpy(u.view(np.int64).copy()), torch.from_numpy(words.view(np.uint8).reshape(-1).copy())

    def global_keys(self, keys, words):
        k = keys.numpy().view(np.uint64)
        w = words.numpy().reshape(-1, 32)
        keep = k != 0
        u, first = np.unique(k[keep], return_index=True)
        self.gkeys, self.gwords = u, w[keep][first].copy().view(np.uint32).reshape(-1, 8)
        self.n_keys = len(u)
        return self.n_keys

    def _kid(self, rec):
        return np.searchsorted(self.gkeys, O.kernel_keys(rec, self.mode))

    def counts_export(self):
        kid = self._kid(self.own)
        solo = (self.own["smem_word"] & SOLO) != 0
        return (torch.from_numpy(np.bincount(kid, minlength=self.n_keys).astype(np.int64)),
                torch.from_numpy(np.bincount(kid[solo], minlength=self.n_keys).astype(np.int64)))

    def counts_import(self, a, b):
        self.launches, self.solo_launches = a.numpy().copy(), b.numpy().copy()

    def samples(self):
        nk = self.n_keys
        own_solo = (self.own["smem_word"] & SOLO) != 0
        so = self.own[own_solo]
        rows = [np.stack([self._kid(so), so["end_ns"] - so["start_ns"], np.zeros(len(so), np.uint64), np.zeros(len(so), np.uint64)], axis=1).astype(np.uint32)]
        tl = np.concatenate([self.halo_rec, self.own])
        nh = len(self.halo_rec)
        s, e = tl["start_ns"], tl["end_ns"]
        solo = (tl["smem_word"] & SOLO) != 0
        ten = tl["smem_word"] >> 24
        kid = self._kid(tl)
        hi = np.searchsorted(s, e, side="left")
        out = []
        for i in np.flatnonzero(~solo):
            for j in range(i + 1, hi[i]):
                if j < nh or solo[j] or ten[j] == ten[i] or not (s[i] < e[j]):
                    continue
                a, b = (i, j) if ten[i] < ten[j] else (j, i)
                out.append((nk + kid[a] * nk + kid[b], e[a] - s[a], e[b] - s[b], max(e[i], e[j]) - s[i]))
        rows.append(np.array(out, dtype=np.uint64).reshape(-1, 4).astype(np.uint32))
        self.smp = np.concatenate(rows)
        return len(self.smp)

    def key_histogram(self):
        nk = self.n_keys
        bits = int(nk + nk * nk).bit_length()
        shift = max(bits - 12, 0)
        b = np.minimum(self.smp[:, 0].astype(np.int64) >> shift, HIST_BINS - 1)
        return torch.from_numpy(np.bincount(b, minlength=HIST_BINS).astype(np.int64)), shift

    def partition(self, splitters, shift, world):
        b = self.smp[:, 0].astype(np.int64) >> shift
        dest = np.zeros(len(b), dtype=np.int64)
        for sp in splitters:
            dest += sp <= b
        order = np.argsort(dest, kind="stable")
        return torch.from_numpy(self.smp[order].view(np.int32).copy())

    def reduce(self, recv):
        smp = recv.numpy().view(np.uint32).reshape(-1, 4)
        order = np.argsort(smp[:, 0], kind="stable")
        self.rs = smp[order]
        key = self.rs[:, 0]
        self.seg = np.flatnonzero(np.r_[True, key[1:] != key[:-1]]) if len(key) else np.zeros(0, np.int64)
        self.cnt = np.diff(np.r_[self.seg, len(key)])
        self.solo_ns = np.full(self.n_keys, np.nan)
        for st, c in zip(self.seg, self.cnt):
            k = int(key[st])
            if k < self.n_keys:
                v = np.sort(self.rs[st: st + c, 1].astype(np.float64))
                self.solo_ns[k] = (v[(c - 1) // 2] + v[c // 2]) * 0.5

    def row_count(self):
        return int(sum(1 for st in self.seg if int(self.rs[st, 0]) >= self.n_keys))

    def solo_export(self):
        return torch.from_numpy(self.solo_ns.copy())

    def solo_import(self, t):
        self.solo_ns = t.numpy().copy()

    def finalize(self):
        nk = self.n_keys
        rows = []
        for st, c in zip(self.seg, self.cnt):
            k = int(self.rs[st, 0])
            if k < nk:
                continue
            ka, kb = divmod(k - nk, nk)
            sa, sb = self.solo_ns[ka], self.solo_ns[kb]
            va, vb = bool(sa > 0), bool(sb > 0)
            r = np.zeros((), dtype=PAIR_ROW_DTYPE)
            r["key_a"], r["key_b"], r["count"], r["flags"] = self.gkeys[ka], self.gkeys[kb], c, int(va) | (int(vb) << 1)
            for tag, lane, solo, ok in (("a", 1, sa, va), ("b", 2, sb, vb)):
                x = np.sort(self.rs[st: st + c, lane].astype(np.float64))
                if ok:
                    r[f"sum_{tag}"] = x.sum() / solo
                    r[f"mean_{tag}"] = x.sum() / solo / c
                    r[f"min_{tag}"], r[f"max_{tag}"] = x[0] / solo, x[-1] / solo
                    r[f"median_{tag}"] = (x[(c - 1) // 2] / solo + x[c // 2] / solo) * 0.5
                else:
                    for f in ("sum", "mean", "min", "max", "median"):
                        r[f"{f}_{tag}"] = np.nan
            sp = np.sort(self.rs[st: st + c, 3].astype(np.float64))
            r["efficiency"] = ((sa + sb) / sp[(c - 1) // 2] + (sa + sb) / sp[c // 2]) * 0.5 if va and vb else np.nan
            r["span_sum_ns"] = int(self.rs[st: st + c, 3].astype(np.uint64).sum())
            rows.append(r)
        self.pair_rows = np.array(rows, dtype=PAIR_ROW_DTYPE) if rows else np.zeros(0, dtype=PAIR_ROW_DTYPE)
        kr = np.zeros(nk, dtype=KEY_ROW_DTYPE)
        kr["key"] = self.gkeys
        kr["name_id"], kr["grid"], kr["block"] = self.gwords[:, 0], self.gwords[:, 1:4], self.gwords[:, 4:7]
        kr["smem"], kr["tenant"] = self.gwords[:, 7] & np.uint32(0x7FFFFF), self.gwords[:, 7] >> 24
        kr["launches"], kr["solo_launches"], kr["solo_ns"] = self.launches, self.solo_launches, self.solo_ns
        self.key_rows = kr

    def tables(self):
        return self.from_bytes(self.key_rows.tobytes()), self.from_bytes(self.pair_rows.tobytes())
