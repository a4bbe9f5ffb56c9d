"""One NCCL rank of tests/test_gpu_parallel.py::test_two_nccl_ranks: python nccl_rank.py <rank> <world> <port> <out dir>."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import numpy as np
import torch
import torch.distributed as dist

from kernel_scheduling_b200 import _lib, parallel, trace
from kernel_scheduling_b200.pair_table import PairTableBuilder
from kernel_scheduling_b200.records import pack_records

rank, world, port, out = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4]
torch.cuda.set_device(rank)
dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
rec = trace.generate(trace.config("c3", 400_000))
lo, hi = parallel.split_windows(len(rec), world)[rank]
stream = torch.cuda.Stream()
with torch.cuda.stream(stream), PairTableBuilder(device=rank, stream=stream.cuda_stream) as b:
    st = parallel.GpuStages(b, torch.from_numpy(rec[lo:hi].view(np.uint8).reshape(-1).copy()).cuda())
    keys, pairs = parallel.run_distributed(parallel.build_steps(st, rank, world))
    torch.cuda.synchronize()
    # the same table through the native driver (exchanges inside the library), twice: the second call reuses every buffer
    session = parallel.NativeSession(b, rank, world)
    window = torch.from_numpy(rec[lo:hi].view(np.uint8).reshape(-1).copy()).cuda()
    torch.cuda.synchronize()
    session.build(window)
    nkeys, npairs = session.build(window)
    # a launch that spans every window, type keys
    n = 4000
    start = np.arange(n, dtype=np.uint64) * 100 + 1000
    dur = np.full(n, 60, dtype=np.uint64)
    tenant = 1 + (np.arange(n) % 2)
    tenant[3], dur[3] = 0, 100 * n
    rec2 = pack_records(tenant, np.ones((n, 3)), np.ones((n, 3)) * 32, np.zeros(n), tenant, np.zeros(n, bool), start, start + dur)
    lo2, hi2 = parallel.split_windows(n, world)[rank]
    window2 = torch.from_numpy(rec2[lo2:hi2].view(np.uint8).reshape(-1).copy()).cuda()
    torch.cuda.synchronize()
    skeys, spairs = session.build(window2, key_type=True)
    # ragged windows: three launches over two ranks, then one launch (the second rank's window is empty)
    tiny_tables, tiny_windows = [], []
    for m in (3, 1):
        lo3, hi3 = parallel.split_windows(m, world)[rank]
        w3 = torch.from_numpy(rec[:m][lo3:hi3].view(np.uint8).reshape(-1).copy()).cuda()
        torch.cuda.synchronize()
        tiny_windows.append(w3)
        tiny_tables.append(session.build(w3))
    # the same builds in stages (every rank owns two or four key ranges; the rows of one are carried to the other GPUs
    # while the next is reduced): forced here, large tables choose it by themselves
    two_stage_ok = True
    for stages in ("2", "4"):
        os.environ["KS_MG_STAGES"] = stages
        staged = [session.build(window), session.build(window), session.build(window2, key_type=True)] + [session.build(w) for w in tiny_windows]
        two_stage_ok = two_stage_ok and all(a[0].tobytes() == b_[0].tobytes() and a[1].tobytes() == b_[1].tobytes()
                                            for a, b_ in zip(staged, [(nkeys, npairs), (nkeys, npairs), (skeys, spairs)] + tiny_tables))
    os.environ["KS_MG_STAGES"] = "1"
    peer_memory = session.peer_memory
    # a bad record in the LAST rank's window: every rank gets the same status from the same call, nobody is left waiting,
    # and the session works afterwards
    bad = rec[lo:hi].copy()
    if rank == world - 1:
        bad["end_ns"][5] = bad["start_ns"][5] - np.uint64(1)
    bad_dev = torch.from_numpy(bad.view(np.uint8).reshape(-1).copy()).cuda()
    torch.cuda.synchronize()
    try:
        session.build(bad_dev)
        status = 0
    except _lib.KsError as e:
        status = e.status
    rkeys, rpairs = session.build(window)
    assert rkeys.tobytes() == nkeys.tobytes() and rpairs.tobytes() == npairs.tobytes()
    session.close()
    # once more with the bulk exchanges forced onto NCCL send/recv
    os.environ["KS_MG_NO_P2P"] = "1"
    session = parallel.NativeSession(b, rank, world)
    assert not session.peer_memory
    ckeys, cpairs = session.build(window)
    session.close()
np.savez(os.path.join(out, f"rank{rank}.npz"), keys=keys, pairs=pairs, nkeys=nkeys, npairs=npairs, skeys=skeys, spairs=spairs, ckeys=ckeys, cpairs=cpairs,
         peer_memory=peer_memory, bad_status=status, two_stage_ok=two_stage_ok, t3keys=tiny_tables[0][0], t3pairs=tiny_tables[0][1], t1keys=tiny_tables[1][0], t1pairs=tiny_tables[1][1])
dist.destroy_process_group()
