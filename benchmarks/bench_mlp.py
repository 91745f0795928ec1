"""Actor-shaped MLP forward (17 -> 256 -> 256 -> 6, tanh): fused three-layer kernel against three GEMM launches,
timed per call inside a CUDA graph of 20 calls (the way the RL trainers run it) and eagerly with CUDA events.

    python benchmarks/bench_mlp.py [--rows 4096,16384]
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def graph_time_us(fn, reps=20, replays=10):
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        fn()
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            for _ in range(reps):
                fn()
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(replays):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * replays)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", default="4096,16384")
    args = ap.parse_args()
    from noeira_b200 import nn
    from noeira_b200.ops import check_status
    from noeira_b200.ops.mlp import mlp3_forward
    nn.manual_seed(0)
    net = nn.Sequential(nn.LinearTanh(17, 256, need_input_grad=False), nn.LinearTanh(256, 256), nn.Linear(256, 6, out_fp32=True)).to("cuda")
    for M in (int(v) for v in args.rows.split(",")):
        x = torch.zeros(M, 24, device="cuda", dtype=torch.bfloat16)
        x[:, :17] = torch.randn(M, 17, device="cuda")
        tf = graph_time_us(lambda: mlp3_forward(x, *net.mods, save=False))
        tfs = graph_time_us(lambda: mlp3_forward(x, *net.mods, save=True))
        tu = graph_time_us(lambda: net.forward(x[:, :17]))
        fl = 2.0 * M * (17 * 256 + 256 * 256 + 256 * 6)
        print(json.dumps({"rows": M, "fused_us": round(tf, 2), "fused_with_saves_us": round(tfs, 2), "three_gemms_us": round(tu, 2),
                          "fused_tflops": round(fl / tf / 1e6, 1), "speedup": round(tu / tf, 2)}))
    check_status()


if __name__ == "__main__":
    main()
