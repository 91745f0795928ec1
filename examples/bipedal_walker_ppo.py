"""PPO on the batched BipedalWalker (CUDA: device rollout of the 2-D rigid-body kernel and the fused update).

    python examples/bipedal_walker_ppo.py [--envs 4096] [--iterations 300]
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--envs", type=int, default=4096)
    ap.add_argument("--iterations", type=int, default=300)
    args = ap.parse_args()
    from noeira_b200.agents.ppo import PPOConfig, PPOTrainer
    from noeira_b200.envs import BipedalWalkerEnv
    env = BipedalWalkerEnv(args.envs, device="cuda", seed=0)
    tr = PPOTrainer(env, PPOConfig(n_envs=args.envs, rollout_len=32, n_epochs=4, n_minibatches=8, hidden=256, entropy_coef=1e-3))
    for it in range(args.iterations):
        m = tr.train_iteration()
        if it % 10 == 9:
            print(f"iteration {it + 1:4d}  reward / step {m['mean_step_reward']:7.3f}  episode return {m['mean_episode_return']:8.1f}  "
                  f"episodes {int(m['episodes'])}")


if __name__ == "__main__":
    main()
