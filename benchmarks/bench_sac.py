"""SAC / TD3 update time on the GPU: glue kernels against the tensor-op form, eager and replayed from a CUDA graph.

    python benchmarks/bench_sac.py [--batch 256] [--iters 200]

Timing: CUDA events around `iters` consecutive updates after 20 warm-up updates (the update is a chain of small launches: no
L2 flush between them, the working set is a few hundred KB).
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def timed(fn, iters):
    for _ in range(20):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--iters", type=int, default=200)
    args = ap.parse_args()
    from noeira_b200.agents.sac import SACConfig, SACTrainer, TD3Config, TD3Trainer
    from noeira_b200 import _native
    g = torch.Generator(device="cuda").manual_seed(0)
    B = args.batch
    batch = (torch.randn(B, 17, device="cuda", generator=g), torch.rand(B, 6, device="cuda", generator=g) * 2 - 1,
             torch.randn(B, device="cuda", generator=g), torch.randn(B, 17, device="cuda", generator=g), torch.zeros(B, device="cuda"))
    for name, mk in (("sac", lambda: SACTrainer(SACConfig(seed=0), device="cuda")), ("td3", lambda: TD3Trainer(TD3Config(seed=0), device="cuda"))):
        row = {"agent": name, "batch": B}
        for label, kernels in (("kernels", True), ("tensor_ops", False)):
            tr = mk()
            tr.use_kernels = kernels
            n0 = _native.launch_count()
            row[f"{label}_eager_ms"] = round(timed(lambda: tr.update(*batch), args.iters), 4)
            row[f"{label}_native_launches_per_update"] = (_native.launch_count() - n0) // (args.iters + 20)
            if name == "sac":
                tr2 = mk()
                tr2.use_kernels = kernels
                row[f"{label}_graph_ms"] = round(timed(lambda: tr2.update_captured(*batch), args.iters), 4)
        print(json.dumps(row))


if __name__ == "__main__":
    main()
