"""LunarLander: device-timed environment throughput and PPO training throughput (the reference's own published PPO
figure is on this environment: 25.4 k env-steps/s on an RTX 5090, docs algorithms/ppo.mdx).

    python benchmarks/bench_lunar.py [--envs 4096] [--steps 200] [--iters 20]
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
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    from noeira_b200.agents.ppo import PPOConfig, PPOTrainer
    from noeira_b200.envs.lunar_lander import LunarLanderEnv
    env = LunarLanderEnv(args.envs, device="cuda", seed=0)
    env.reset_batch()
    act = torch.rand(args.envs, 2, device="cuda") * 2 - 1
    for _ in range(10):
        env.step_batch(act)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(args.steps):
        env.step_batch(act)
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / args.steps
    print(json.dumps({"what": "env step only", "envs": args.envs, "ms_per_batched_step": round(ms, 4),
                      "env_steps_per_s": round(args.envs / ms * 1e3)}))
    env = LunarLanderEnv(args.envs, device="cuda", seed=0)
    agent = PPOTrainer(env, PPOConfig(n_envs=args.envs, rollout_len=32, n_epochs=4, n_minibatches=8))
    for _ in range(3):
        agent.train_iteration(read_metrics=False)
    torch.cuda.synchronize()
    s.record()
    for _ in range(args.iters):
        agent.train_iteration(read_metrics=False)
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / args.iters
    m = agent.train_iteration()
    print(json.dumps({"what": "PPO iteration (rollout 32, 4 epochs x 8 minibatches)", "envs": args.envs, "ms_per_iteration": round(ms, 3),
                      "env_steps_per_s": round(args.envs * 32 / ms * 1e3), "reference_published_env_steps_per_s": 25400,
                      "mean_episode_return": m.get("mean_episode_return")}))


if __name__ == "__main__":
    main()
