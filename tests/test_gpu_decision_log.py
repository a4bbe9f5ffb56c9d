"""GPU: the decision-log analytics (device parse, radix-sort grouping, segmented statistics and histograms) against the
pandas oracle, on a synthetic daemon log + agent logs in the reference's formats."""
import numpy as np
import pytest

from kernel_scheduling_b200 import _lib, decision_log
from oracle import decision_log_oracle as DO

pytestmark = pytest.mark.gpu

DECISION_HEADER = ("batch_id\tbatch_size\tbatch_pos\tdecision_ns\tpost_ns\tpid\tkernel_id\tarrival_seq\tkernel_name\tlayer_tag\t"
                   "request_ns\tqueue_wait_us\tend_ns\tn_pending\tpending_pids\tinflight_slot\tkernel_base\tgrid\tblock\tmodel\n")
AGENT_HEADER = ("kernel_id\tkernel_us\tprefetch_us\tprefetch_to_kernel_gap_us\thook_tag\tprefetch_bytes\tprefetched_tensors\targs_check\tkernel_name\t"
                "start_ns\tend_ns\tbatch_id\tbatch_size\tbatch_pos\tblock\tmodel\tgrid\n")


def synth_logs(n=6000, seed=3, crlf=False):
    rng = np.random.default_rng(seed)
    pids = {4101: "qwen", 4202: "whisper"}
    bases = ["gemm_kernel", "softmax_warp", "layer_norm", "vectorized_elementwise_kernel", "rope", "conv1d_fwd"]
    blocks = ["(128, 1, 1)", "(256, 1, 1)", "(32, 8, 1)"]
    next_kid = {p: 0 for p in pids}
    agent_rows = {p: [] for p in pids}
    lines, t, batch = [], 10**12, 0
    while len(lines) < n:
        batch += 1
        size = int(rng.choice([1, 1, 1, 2, 2, 3, 20]))
        decision_ns = t
        for pos in range(size):
            pid = int(rng.choice(list(pids)))
            kid = next_kid[pid]
            next_kid[pid] += 1
            base, block = bases[int(rng.integers(len(bases)))], blocks[int(rng.integers(len(blocks)))]
            request = t - int(rng.integers(1_000, 3_000_000))
            post = t + pos * 700
            wait = "" if rng.random() < 0.03 else f"{(post - request) / 1000.0:.3f}"
            start, dur = post + 2000, int(rng.integers(2_000, 400_000))
            end = "" if rng.random() < 0.02 else str(start + dur)
            lines.append(f"{batch}\t{size}\t{pos}\t{decision_ns}\t{post}\t{pid}\t{kid}\t{len(lines)}\tvoid {base}<float>(float*)\t-\t{request}\t{wait}\t{end}\t"
                         f"{int(rng.integers(1, 5))}\t4101,4202\t{int(rng.integers(0, 8))}\t{base}\t({int(rng.integers(1, 500))}, 1, 1)\t{block}\t{pids[pid]}")
            if rng.random() > 0.05:  # some launches never made it into the agent's log
                e = "" if rng.random() < 0.02 else str(start + dur)
                agent_rows[pid].append(f"{kid}\t{dur / 1000:.3f}\t\t\t-\t0\t\t-\tvoid {base}<float>(float*)\t{start}\t{e}\t{batch}\t{size}\t{pos}\t{block}\t{pids[pid]}\t(8, 1, 1)")
        t += int(rng.integers(5_000, 900_000))
    nl = "\r\n" if crlf else "\n"
    decision = (DECISION_HEADER.replace("\n", nl) + nl.join(lines) + nl).encode()
    agents = {p: (AGENT_HEADER.replace("\n", nl) + nl.join(r) + nl).encode() for p, r in agent_rows.items()}
    return decision, agents


@pytest.mark.parametrize("crlf", [False, True])
def test_decision_log_analytics_match_the_pandas_oracle(builder, crlf):
    decision, agents = synth_logs(crlf=crlf)
    got = decision_log.analyse(decision, agents, builder)
    want = DO.analyse(decision, agents)
    assert len(got["key"]) == len(want) == 36  # 2 models x 6 kernels x 3 blocks
    index = {(m, k, tuple(int(x) for x in b)): i for i, (m, k, b) in enumerate(zip(got["model"], got["kernel"], got["block"]))}
    assert len(index) == 36
    for _, w in want.iterrows():
        i = index[(w["model"], w["kernel"], tuple(w["block"]))]
        for c in ("rows", "wait_rows", "wait_ns_sum", "wait_ns_min", "wait_ns_max", "dur_alone_rows", "dur_gang_rows"):
            assert int(got[c][i]) == int(w[c]), c
        for c in ("wait_ns_median", "dur_alone_median_ns", "dur_gang_median_ns"):
            assert np.array_equal(np.float64(got[c][i]), np.float64(w[c]), equal_nan=True), c
        assert np.array_equal(got["wait_hist"][i], w["wait_hist"]) and np.array_equal(got["batch_hist"][i], w["batch_hist"])
    assert int(got["rows"].sum()) == int(want["rows"].sum()) >= 6000


def test_tsv_extract_kinds(builder):
    text = (b"a\tb\tc\td\n" b"12\t3.5\t(1, 2, 3)\tfoo\n" b"\t0.001\t4,5,6\t\n" b"7.0\tx\t(1,2)\tfoo\r\n" b"99\t12.3456\t(2097152, 1, 1)\tbar")
    a, b, c, d, span = builder.tsv_extract(text, [(0, _lib.COL_U64), (1, _lib.COL_MILLI), (2, _lib.COL_DIMS), (3, _lib.COL_HASH), (3, _lib.COL_SPAN)])
    none = 0xFFFFFFFFFFFFFFFF
    assert a.tolist() == [12, none, 7, 99]
    assert b.tolist() == [3500, 1, none, 12345]
    assert c.tolist() == [1 | 2 << 21 | 3 << 42, 4 | 5 << 21 | 6 << 42, none, none]
    assert d[0] == d[2] and d[0] != d[3] and d[1] != d[0]
    assert [text[int(s) >> 20: (int(s) >> 20) + (int(s) & 0xFFFFF)] for s in span] == [b"foo", b"", b"foo", b"bar"]
    # a column the line does not have, and an empty text
    assert builder.tsv_extract(b"h1\th2\nx\n", [(1, _lib.COL_U64)])[0].tolist() == [none]
    assert len(builder.tsv_extract(b"", [(0, _lib.COL_U64)])[0]) == 0
    assert len(builder.tsv_extract(b"only a header\n", [(0, _lib.COL_U64)])[0]) == 0


def test_segment_hist(builder):
    rng = np.random.default_rng(1)
    v = rng.integers(0, 1 << 20, 5000).astype(np.uint32)
    off = np.array([0, 0, 10, 3000, 5000], dtype=np.uint64)
    got = builder.segment_hist(v, off, 33, log2_bins=True)
    for s in range(4):
        seg = v[int(off[s]): int(off[s + 1])]
        want = np.bincount([int(x).bit_length() for x in seg], minlength=33)
        assert np.array_equal(got[s], want)
    lin = builder.segment_hist(np.minimum(v, 40).astype(np.uint32), off, 17)
    assert np.array_equal(lin[3], np.bincount(np.minimum(np.minimum(v[3000:], 40), 16), minlength=17))
