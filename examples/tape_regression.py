"""The eager tape mode of ``nn``: a network whose wiring is plain code with run-time shapes, an ``nn`` module used as one
node, the arena optimizer of ``nn`` stepping the tape's parameters (CPU or CUDA).

    python examples/tape_regression.py [--device cpu] [--steps 400]
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--steps", type=int, default=400)
    args = ap.parse_args()
    import torch
    from noeira_b200 import nn
    from noeira_b200.experimental.functional import F, Tape, TapeAdam
    tape = Tape(device=args.device, seed=0)
    w1, b1 = tape.param(8, 64, name="w1"), tape.zeros(1, 64, name="b1")
    norm = tape.module(nn.LayerNorm(64), "norm")                   # an nn module as one node of the tape
    w2, b2 = tape.param(64, 8, "xavier", name="w2"), tape.zeros(1, 8, name="b2")
    opt = TapeAdam(tape, lr=3e-3)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(512, 8, generator=g).to(args.device)
    y = torch.sin(x) * x.roll(1, 1)
    for step in range(args.steps):
        tape.reset()
        h = norm(F.linear(tape.constant(x), w1, b1, "tanh"))
        loss = F.mse(F.linear(h, w2, b2), y)
        loss.backward()
        opt.step()
        if step % 50 == 0 or step == args.steps - 1:
            print(f"step {step:4d}  loss {loss.item():.5f}  nodes on the tape {len(tape)}")


if __name__ == "__main__":
    main()
