"""Device-timed throughput of the fused physics env step (env-steps/s) for the planar chain.

    python benchmarks/bench_physics.py [--envs 4096] [--steps 200]
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--envs", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--model", default="planar_chain")
    args = ap.parse_args()
    from noeira_b200.envs import HalfCheetahEnv, PlanarChainEnv
    env = (PlanarChainEnv if args.model == "planar_chain" else HalfCheetahEnv)(args.envs, seed=0)
    env.reset_batch()
    a = torch.rand(args.envs, env.act_dim, device="cuda") * 2 - 1
    for _ in range(20):
        env.step_batch(a)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(args.steps):
        env.step_batch(a)
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / args.steps
    print(json.dumps({"model": args.model, "envs": args.envs, "ms_per_env_step_batch": round(ms, 4),
                      "env_steps_per_s": round(args.envs / ms * 1e3), "substeps_per_s": round(5 * args.envs / ms * 1e3),
                      "finite": bool(torch.isfinite(env.obs).all().item())}))


if __name__ == "__main__":
    main()
