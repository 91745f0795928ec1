"""Device-timed leaf kernels outside the GEMM / attention benchmarks: LayerNorm / RMSNorm forward + backward, Conv2D forward
(implicit GEMM against the patch-matrix path), BatchNorm2D forward + backward, max-pool, the ray-traced camera.

    python benchmarks/bench_layers.py [--iters 10] [--only norm|conv|bn|pool|ray]
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def timeit(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--only", default="")
    args = ap.parse_args()
    from noeira_b200 import nn
    from noeira_b200.ops import check_status
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    peak = 6552.0
    try:
        peak = json.load(open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")))["hbm_gbs"]
    except Exception:  # noqa: BLE001
        pass
    want = lambda k: not args.only or args.only == k

    if want("norm"):
        for cls, M, D in ((nn.LayerNorm, 196608, 768), (nn.RMSNorm, 16384, 2048)):
            ln = cls(D).to("cuda")
            x = torch.randn(M, D, device="cuda").bfloat16()
            t = timeit(lambda: ln.forward(x), args.iters, flush)
            y = ln.forward(x)
            dy = torch.randn_like(y)
            tb = timeit(lambda: ln.vjp(dy), args.iters, flush)
            gb = 2 * M * D * 2 / 1e9
            print(json.dumps({"op": cls.__name__, "shape": [M, D], "fwd_ms": round(t, 4), "fwd_gbs": round(gb / t * 1e3, 1),
                              "fwd_frac_of_measured_copy": round(gb / t * 1e3 / peak, 3), "bwd_ms": round(tb, 4),
                              "bwd_gbs": round(1.5 * gb / tb * 1e3, 1)}))
    if want("conv"):
        for ic, oc, H, W in ((64, 64, 120, 160), (128, 128, 60, 80), (256, 256, 30, 40)):
            a = nn.Conv2D(ic, oc, 3, 1, 1, bias=False).to("cuda")
            b = nn.Conv2D(ic, oc, 3, 1, 1, bias=False).to("cuda")
            b.implicit_gemm = False
            a.force_implicit = True
            x = torch.randn(16, H, W, ic, device="cuda").bfloat16()
            ti = timeit(lambda: a.forward(x), args.iters, flush)
            tp = timeit(lambda: b.forward(x), args.iters, flush)
            fl = 2.0 * 16 * H * W * oc * 9 * ic
            print(json.dumps({"op": "conv3x3 fwd", "shape": [16, H, W, ic, oc], "implicit_ms": round(ti, 4),
                              "implicit_tflops": round(fl / ti / 1e9, 1), "patch_matrix_ms": round(tp, 4),
                              "patch_matrix_tflops": round(fl / tp / 1e9, 1)}))
    if want("bn"):
        bn = nn.BatchNorm2D(64, relu=True).to("cuda")
        x = torch.randn(16, 120, 160, 64, device="cuda").bfloat16()
        t = timeit(lambda: bn.forward(x), args.iters, flush)
        y = bn.forward(x)
        dy = torch.randn_like(y)
        tb = timeit(lambda: bn.vjp(dy), args.iters, flush)
        gb = x.numel() * 2 / 1e9
        print(json.dumps({"op": "BatchNorm2D+ReLU", "shape": list(x.shape), "fwd_ms": round(t, 4), "fwd_gbs": round(3 * gb / t * 1e3, 1),
                          "bwd_ms": round(tb, 4), "bwd_gbs": round(5 * gb / tb * 1e3, 1)}))
    if want("pool"):
        mp = nn.MaxPool2D()
        x = torch.randn(16, 240, 320, 64, device="cuda").bfloat16()
        t = timeit(lambda: mp.forward(x), args.iters, flush)
        y = mp.forward(x)
        dy = torch.randn_like(y)
        tb = timeit(lambda: mp.vjp(dy), args.iters, flush)
        print(json.dumps({"op": "MaxPool2D 3x3/2", "shape": list(x.shape), "fwd_ms": round(t, 4), "bwd_ms": round(tb, 4)}))
    if want("ray"):
        from noeira_b200.envs import PlanarChainEnv
        from noeira_b200.physics.raytrace import BatchedCameraRenderer, Camera
        env = PlanarChainEnv(1024, seed=0)
        env.reset_batch()
        xpos, xmat = env.engine.body_poses()
        r = BatchedCameraRenderer(env.engine.model, [Camera((0.3, -2.5, 0.9), (0.3, 0.0, 0.4))], 64, 64)
        t = timeit(lambda: r.render(xpos, xmat), args.iters, flush)
        print(json.dumps({"op": "raytrace 64x64", "worlds": 1024, "ms": round(t, 4), "mpixels_per_s": round(1024 * 4096 / t / 1e3, 1),
                          "frames_per_s": round(1024 / t * 1e3)}))
    check_status()


if __name__ == "__main__":
    main()
