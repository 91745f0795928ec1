"""gloo rank of tests/test_distributed_cpu.py::test_gloo_processes_match_simulator."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

if __name__ == "__main__":
    dist.init_process_group("gloo")
    from noeira_b200.parallel.fibers import DistComm
    from test_distributed_cpu import _train
    strategy = os.environ.get("STRATEGY", "ddp")
    v, _ = _train(DistComm(), strategy)
    torch.save(v, os.environ["OUT"] + str(dist.get_rank()))
    dist.destroy_process_group()
