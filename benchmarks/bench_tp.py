"""Fused tensor-parallel kernels (all-gather→GEMM, GEMM→reduce-scatter) against NCCL + the unfused GEMM at the four
layer shapes of the world model, device-timed, max over ranks, with the roofline of each shape.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29515 \\
        benchmarks/bench_tp.py [--ms 16512] [--iters 10]

Roofline of one call on one GPU = the slower of
  compute   2·(N·Ms)·n·k FLOP at the measured sustained cuBLAS bf16 rate (MEASURED_PEAKS.json, 1399.6 TFLOP/s), and
  link      (N-1)·Ms·width·2 bytes that must enter (all-gather: width = k) or leave (reduce-scatter: width = n) this
            GPU over NVLink at the measured 770 GB/s per direction.
`frac` = roofline time / measured time.  Each timed call is preceded by an L2 flush (256 MB write) outside the event pair.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
LINK_GBS, GEMM_TFLOPS = 770.0, 1399.6


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ms", type=int, default=16512, help="rows per rank (one padded world-model sequence)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--dim", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--ff", type=int, default=5632)
    args = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from noeira_b200.ops import check_status
    from noeira_b200.parallel.tp import NcclTP, TPLinearContext
    ms, d, hd = args.ms, args.dim, 128
    hq, hkv, ffl = args.heads // world, max(args.kv_heads // world, 1), args.ff // world
    shapes = [("qkv  (ag)", "ag", d, (hq + 2 * hkv) * hd), ("out  (rs)", "rs", hq * hd, d),
              ("up   (ag)", "ag", d, 2 * ffl), ("down (rs)", "rs", ffl, d)]
    base = NcclTP(world, rank)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(1 + rank)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(args.iters):
            flush.zero_()
            if world > 1:
                dist.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        ts.sort()
        t = torch.tensor([ts[len(ts) // 2]], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for name, kind, k, n in shapes:
        ctx = TPLinearContext(world, rank, ms, k, n, kind)
        w = (torch.randn(k, n, device="cuda", generator=g) * 0.02).bfloat16()
        if kind == "ag":
            x = torch.randn(ms, k, device="cuda", generator=g).bfloat16()
            ctx.x_shard.copy_(x)
            fused = lambda: ctx.ag_gemm(w, True)
            lib = lambda: base.ag_gemm(x, w, True)
            link_bytes = (world - 1) * ms * k * 2
        else:
            a = torch.randn(world * ms, k, device="cuda", generator=g).bfloat16()
            res = torch.randn(ms, n, device="cuda", generator=g).bfloat16()
            fused = lambda: ctx.gemm_rs(a, w, True, residual=res)
            lib = lambda: base.gemm_rs(a, w, True, residual=res)
            link_bytes = (world - 1) * ms * n * 2
        t_f, t_l = timed(fused), timed(lib)
        flops = 2.0 * world * ms * n * k
        t_c, t_n = flops / (GEMM_TFLOPS * 1e12) * 1e3, link_bytes / (LINK_GBS * 1e9) * 1e3
        roof = max(t_c, t_n)
        if rank == 0:
            print(json.dumps({"layer": name.strip(), "world": world, "rows": world * ms, "k": k, "n": n,
                              "fused_ms": round(t_f, 4), "nccl_plus_gemm_ms": round(t_l, 4), "speedup_vs_nccl": round(t_l / t_f, 3),
                              "compute_bound_ms": round(t_c, 4), "link_bound_ms": round(t_n, 4),
                              "limiter": "compute" if t_c >= t_n else "nvlink", "frac_of_roofline": round(roof / t_f, 3),
                              "tflops": round(flops / t_f / 1e9, 1), "link_gbs": round(link_bytes / t_f / 1e6, 1)}), flush=True)
        del ctx
    check_status()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
