"""TD-MPC2 on Pendulum: latent world model + Q ensemble, actions chosen by planning in latent space.

    python examples/tdmpc2_pendulum.py [--steps 20000] [--device cpu]
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20000)
    ap.add_argument("--device", default="cpu")
    args = ap.parse_args()
    from noeira_b200.agents.tdmpc2 import TDMPC2Agent, TDMPC2Config, run_tdmpc2
    from noeira_b200.envs import PendulumEnv
    env = PendulumEnv(8, device=args.device, seed=0)
    ag = TDMPC2Agent(TDMPC2Config(obs_dim=3, act_dim=1), n_envs=8, device=args.device)
    done = 0
    while done < args.steps:
        rets = run_tdmpc2(env, ag, total_env_steps=1600, seed_steps=1600 if done == 0 else 0)
        done += 1600
        print(f"env steps {done:6d}  episodes {len(rets)}  mean return {sum(rets) / max(len(rets), 1):8.1f}  {ag.last}")


if __name__ == "__main__":
    main()
