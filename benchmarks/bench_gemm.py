"""Device-timed GEMM throughput of the tcgen05 kernel vs. cuBLAS (torch.matmul) on the same shapes.

    python benchmarks/bench_gemm.py [--shapes 8192x8192x8192,4096x4096x4096] [--iters 20] [--two-cta 0|1|2]

Timing: CUDA events on the launching stream, 5 warm-ups, an L2 flush (write of a 256 MB buffer)
between timed iterations, median of `iters`.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def timeit(fn, iters, flush):
    for _ in range(5):
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
    ap.add_argument("--shapes", default="8192x8192x8192,4096x4096x4096,16384x256x256,16384x5632x2048,2048x2048x16384")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--layout", default="nt", help="nt: B [N,K]; nn: B [K,N]; tn: A [K,M], B [K,N]")
    ap.add_argument("--two-cta", type=int, default=0, help="0 = by size, 1 = one-CTA tiles only, 2 = CTA-pair tiles")
    ap.add_argument("--no-lib", action="store_true", help="skip the cuBLAS comparison (profiling captures)")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "tf32"], help="tf32: fp32 operands on the TF32 tensor-core path")
    args = ap.parse_args()
    from noeira_b200.ops import check_status, gemm
    from noeira_b200.ops.gemm import set_two_cta_mode
    set_two_cta_mode(args.two_cta)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(os.path.dirname(__file__), "..", "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak = peaks.get("bf16_tflops", 1590.0)          # TF32 runs at half the bf16 rate: its fraction is taken against peak / 2
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for sh in args.shapes.split(","):
        M, N, K = (int(x) for x in sh.split("x"))
        a_mn = args.layout == "tn"
        b_mn = args.layout in ("nn", "tn")
        dt = torch.bfloat16 if args.dtype == "bf16" else torch.float32
        torch.backends.cuda.matmul.allow_tf32 = args.dtype == "tf32"        # the library comparison uses TF32 too
        a = (torch.randn((K, M) if a_mn else (M, K), device="cuda") * 0.1).to(dt)
        b = (torch.randn((K, N) if b_mn else (N, K), device="cuda") * 0.1).to(dt)
        out = torch.empty(M, N, device="cuda", dtype=dt)
        A = a.t() if a_mn else a
        B = b if b_mn else b.t()
        t_ours = timeit(lambda: gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out, bn=args.bn), args.iters, flush)
        check_status()
        t_lib = float("nan") if args.no_lib else timeit(lambda: torch.matmul(A, B, out=out), args.iters, flush)
        fl = 2.0 * M * N * K
        print(json.dumps({"shape": sh, "layout": args.layout, "dtype": args.dtype, "ours_ms": round(t_ours, 4), "cublas_ms": round(t_lib, 4),
                          "ours_tflops": round(fl / t_ours / 1e9, 1), "cublas_tflops": round(fl / t_lib / 1e9, 1),
                          "frac_of_measured_peak": round(fl / t_ours / 1e9 / (peak if args.dtype == "bf16" else peak / 2), 3)}))


if __name__ == "__main__":
    main()
