"""One gloo rank of tests/test_parallel_cpu.py::test_two_gloo_ranks: python gloo_rank.py <rank> <world> <port> <out dir>."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import numpy as np
import torch.distributed as dist

from kernel_scheduling_b200 import parallel, trace
from tests.fake_stages import FakeStages

rank, world, port, out = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4]
dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
rec = trace.generate(trace.config("c3", 2500))
lo, hi = parallel.split_windows(len(rec), world)[rank]
keys, pairs = parallel.run_distributed(parallel.build_steps(FakeStages(rec[lo:hi]), rank, world))
np.savez(os.path.join(out, f"rank{rank}.npz"), keys=keys, pairs=pairs)
dist.destroy_process_group()
