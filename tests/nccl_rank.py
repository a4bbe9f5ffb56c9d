"""One NCCL rank of tests/test_gpu_parallel.py::test_two_nccl_ranks: python nccl_rank.py <rank> <world> <port> <out dir>."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import numpy as np
import torch
import torch.distributed as dist

from kernel_scheduling_b200 import parallel, trace
from kernel_scheduling_b200.pair_table import PairTableBuilder

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
np.savez(os.path.join(out, f"rank{rank}.npz"), keys=keys, pairs=pairs)
dist.destroy_process_group()
