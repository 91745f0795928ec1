"""PPO on 4096 GPU-batched planar-chain environments (needs a B200): rollout, GAE and the minibatch updates are CUDA graphs.

    python examples/ppo_planar_chain.py [--iterations 200] [--envs 4096] [--checkpoint ppo_chain.ckpt]
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iterations", type=int, default=200)
    ap.add_argument("--envs", type=int, default=4096)
    ap.add_argument("--checkpoint", default="")
    ap.add_argument("--runs", default="runs")
    args = ap.parse_args()
    from noeira_b200 import core
    from noeira_b200.agents.ppo import PPOConfig, PPOTrainer
    from noeira_b200.envs import PlanarChainEnv
    env = PlanarChainEnv(args.envs, seed=0)
    tr = PPOTrainer(env, PPOConfig(n_envs=args.envs))
    with core.RunContext(args.runs, "examples", "ppo-chain", {"envs": args.envs}) as run:
        for it in range(args.iterations):
            m = tr.train_iteration()
            if it % 10 == 0:
                run.log(it, {k: v for k, v in m.items() if v == v})
                print(it, {k: round(v, 4) for k, v in m.items() if v == v})
        if args.checkpoint:
            tr.save(args.checkpoint)


if __name__ == "__main__":
    main()
