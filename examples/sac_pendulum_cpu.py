"""SAC on the batched Pendulum swing-up, entirely on the CPU (fp32 explicit-backward path), logged to a run directory.

    python examples/sac_pendulum_cpu.py [--steps 30000] [--envs 8]
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=30000)
    ap.add_argument("--envs", type=int, default=8)
    ap.add_argument("--runs", default="runs")
    args = ap.parse_args()
    from noeira_b200 import core
    from noeira_b200.agents.sac import SACAgent, SACConfig
    from noeira_b200.envs import PendulumEnv
    env = PendulumEnv(args.envs, seed=0)
    cfg = SACConfig(obs_dim=3, act_dim=1, hidden=128, batch=128)
    agent = SACAgent(env, cfg, capacity=100_000, learning_starts=1000)
    with core.RunContext(args.runs, "examples", "sac-pendulum", {"steps": args.steps, "envs": args.envs}) as run:
        agent.train(args.steps, logger=run, log_every=2000)
        ret = float(env.ep_stats[0] / max(float(env.ep_stats[1]), 1.0))
        print(f"mean episode return over training: {ret:.1f}   run dir: {run.dir}")


if __name__ == "__main__":
    main()
