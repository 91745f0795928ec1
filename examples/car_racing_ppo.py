"""PPO on the batched CarRacing environment from its state observation with look-ahead track points (CUDA: the fused
tire-model step kernel under the on-device PPO update), with the pure-pursuit driver's return printed as a yardstick.

    python examples/car_racing_ppo.py [--envs 2048] [--iterations 200]
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--envs", type=int, default=2048)
    ap.add_argument("--iterations", type=int, default=200)
    args = ap.parse_args()
    import torch
    from noeira_b200.agents.ppo import PPOConfig, PPOTrainer
    from noeira_b200.envs import CarRacingEnv, scripted_driver
    ref = CarRacingEnv(256, device="cuda", seed=1, lookahead=8)
    ref.reset_batch()
    total = torch.zeros(256, device="cuda")
    for _ in range(1000):
        _, r, _, _ = ref.step_batch(scripted_driver(ref), auto_reset=False)
        total += r
    print(f"scripted driver: return over 1000 steps {float(total.mean()):.1f}, tiles visited {float(ref.visited_fraction().mean()):.2f}")
    env = CarRacingEnv(args.envs, device="cuda", seed=0, lookahead=8)
    # the environment step is one kernel launch that works in place, so the whole rollout replays from a CUDA graph
    tr = PPOTrainer(env, PPOConfig(n_envs=args.envs, rollout_len=64, n_epochs=4, n_minibatches=8, hidden=256, entropy_coef=1e-3))
    for it in range(args.iterations):
        m = tr.train_iteration()
        if it % 10 == 9:
            print(f"iteration {it + 1:4d}  reward / step {m['mean_step_reward']:7.3f}  episode return {m['mean_episode_return']:8.1f}  "
                  f"episodes {int(m['episodes'])}")


if __name__ == "__main__":
    main()
