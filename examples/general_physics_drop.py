"""The general rigid-body engine: a free box with a ball-jointed arm dropped on the ground plane, read through sensors.

    python examples/general_physics_drop.py [--solver newton|pgs] [--integrator euler|implicit|rk4]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

XML = """<mujoco><compiler angle="radian"/><option timestep="0.002"/>
  <worldbody><geom type="plane" pos="0 0 0" size="5 5 0.1"/>
    <body name="base" pos="0 0 0.6"><freejoint name="root"/><geom type="box" size="0.2 0.1 0.05"/>
      <body name="arm" pos="0.2 0 0.05"><joint type="ball" name="shoulder"/><geom type="capsule" fromto="0 0 0 0.3 0 0" size="0.03"/>
        <body name="hand" pos="0.3 0 0"><joint type="hinge" axis="0 1 0" range="-1 1" name="wrist"/><geom type="sphere" size="0.04"/></body>
      </body></body></worldbody>
  <actuator><motor joint="wrist" gear="1"/></actuator></mujoco>"""


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--solver", default="newton")
    ap.add_argument("--integrator", default="euler")
    ap.add_argument("--envs", type=int, default=4)
    args = ap.parse_args()
    from noeira_b200.physics import general as G
    from noeira_b200.physics.mjcf import from_mjcf
    model = from_mjcf(XML, general=True)
    sim = G.GeneralSim(model, args.envs, integrator=args.integrator, solver=args.solver)
    sim.qvel[:, 3:6] = torch.randn(args.envs, 3, dtype=torch.float64)             # each copy tumbles differently
    for step in range(1, 1001):
        sim.step(torch.full((args.envs, 1), 0.2))
        if step % 100 == 0:
            s = sim.sensors(0)
            T, U = G.energy(model, sim.qpos, sim.qvel)
            print(f"t={step * 0.002:5.2f}s  base z {s['framepos'][0, 2]:.3f}  touch {s['touch'][0]:7.2f} N  "
                  f"accelerometer z {s['accelerometer'][0, 2]:6.2f}  energy {float(T[0] + U[0]):8.3f}")


if __name__ == "__main__":
    main()
