"""CarRacing on the GPU: the fused step kernel, the whole environment step (kernel + masked reset + observation), the camera
kernel, and PPO iterations on top of it.

    python benchmarks/bench_car_racing.py [--envs 4096] [--iters 100] [--res 96] [--ppo-iters 0]

Timing: CUDA events around `iters` consecutive calls after 10 warm-up calls.  The state of 4096 lanes is 4.4 MB and a batch of
96 x 96 frames 151 MB (larger than L2), so the camera figure includes its DRAM writes.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def timed(fn, iters):
    for _ in range(10):
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
    ap.add_argument("--envs", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--res", type=int, default=96)
    ap.add_argument("--ppo-iters", type=int, default=0)
    ap.add_argument("--graphs", type=int, default=1, help="replay the PPO rollout and update from CUDA graphs")
    args = ap.parse_args()
    from noeira_b200.envs.car_racing import CarRacingEnv, scripted_driver
    env = CarRacingEnv(args.envs, device="cuda", seed=0, lookahead=8)
    env.reset_batch()
    for _ in range(50):                                           # spread the cars along their tracks
        env.step_batch(scripted_driver(env))
    a = scripted_driver(env)
    out = {"envs": args.envs, "res": args.res}
    out["step_kernel_ms"] = timed(lambda: env._dynamics(env.state, a), args.iters)
    out["env_step_ms"] = timed(lambda: env.step_batch(a), args.iters)
    out["render_ms"] = timed(lambda: env.render(args.res), args.iters)
    out["render_uint8_ms"] = timed(lambda: env.render(args.res, uint8=True), args.iters)
    out["env_steps_per_s"] = args.envs / out["env_step_ms"] * 1e3
    out["frames_per_s"] = args.envs / out["render_ms"] * 1e3
    out["render_write_gbs"] = args.envs * args.res * args.res * 4 / out["render_ms"] / 1e6
    if args.ppo_iters:
        from noeira_b200.agents.ppo import PPOConfig, PPOTrainer
        tr = PPOTrainer(env, PPOConfig(n_envs=args.envs, rollout_len=32, n_epochs=4, n_minibatches=8, hidden=256, entropy_coef=1e-3,
                                       use_cuda_graphs=bool(args.graphs)))
        curve = []
        for it in range(args.ppo_iters):
            m = tr.train_iteration()
            if it % max(1, args.ppo_iters // 8) == 0 or it == args.ppo_iters - 1:
                curve.append((it, round(float(m["mean_step_reward"]), 4)))
        out["graphs"] = bool(args.graphs)
        out["ppo_iteration_ms"] = timed(lambda: tr.train_iteration(read_metrics=False), 5)
        out["ppo_env_steps_per_s"] = args.envs * 32 / out["ppo_iteration_ms"] * 1e3
        out["ppo_reward_per_step"] = curve
    print(json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in out.items()}))


if __name__ == "__main__":
    main()
