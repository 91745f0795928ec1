"""Rainbow (noisy dueling C51, 3-step returns, prioritised replay) on a two-action CartPole.

    python examples/rainbow_cartpole.py [--steps 40000] [--device cpu]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


class TwoActionCartPole:
    """The continuous-force CartPole of the env zoo driven by two pushes."""

    def __init__(self, n, device, seed=0):
        from noeira_b200.envs import CartPoleEnv
        self.env = CartPoleEnv(n, device=device, seed=seed)
        self.n_envs = n

    def __getattr__(self, k):
        return getattr(self.env, k)

    def step_batch(self, a):
        return self.env.step_batch((a.float() * 2 - 1).reshape(-1, 1))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=40000)
    ap.add_argument("--device", default="cpu")
    args = ap.parse_args()
    from noeira_b200.agents.rainbow import RainbowConfig, RainbowTrainer, run_rainbow
    env = TwoActionCartPole(16, args.device)
    tr = RainbowTrainer(RainbowConfig(obs_dim=4, n_actions=2, hidden=128, n_atoms=51, v_min=0.0, v_max=100.0, gamma=0.99), device=args.device)
    seen = [0]

    def log(step, finished):
        if len(finished) >= seen[0] + 50:
            seen[0] = len(finished)
            print(f"step {step:7d}  episodes {len(finished):5d}  mean return of the last 50: {sum(finished[-50:]) / 50:.1f}")

    run_rainbow(env, tr, args.steps, log=log)


if __name__ == "__main__":
    main()
