"""Fused P2P all-reduce (push / one-shot / two-shot) vs NCCL, per bucket size, device-timed, max over ranks.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29512 \\
        benchmarks/bench_allreduce.py [--max-mb 256] [--adam]

Roofline: with reduction inside the switch an all-reduce must move (N-1)/N · bytes in each direction per GPU
(`*_frac_of_roofline`); without it (reduce-scatter then all-gather over peer loads, what these kernels do) the
bandwidth-optimal bound is 2(N-1)/N · bytes per direction (`*_frac_of_p2p_bound`); both at the measured 770 GB/s.  `--adam` times the fused reduce+AdamW kernel against NCCL all-reduce followed
by the single-GPU arena AdamW kernel.
"""
import argparse
import ctypes
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
LINK_GBS = 770.0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-mb", type=int, default=256)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--adam", action="store_true")
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    table(rank, world, args.max_mb, args.iters, args.adam, emit=True)
    dist.barrier()
    dist.destroy_process_group()


def table(rank, world, max_mb, iters, adam, emit=True):
    """Time every form at sizes 64 KB … max_mb (x4 steps) in the current process group; returns the rows."""
    import types
    args = types.SimpleNamespace(max_mb=max_mb, iters=iters, adam=adam)
    from noeira_b200._native import check, cuda_lib, ptr, stream_ptr
    from noeira_b200.ops.status import check_status, device_status
    from noeira_b200.parallel.symm import SIGNAL_PAD_WORDS, SymmetricHeap
    lib = cuda_lib()
    max_n = args.max_mb * (1 << 20) // 4
    heap = SymmetricHeap(2 * max_n * 4 + 8192)
    grd, red = heap.tensor(max_n, torch.float32), heap.tensor(max_n, torch.float32)
    sig = heap.tensor(SIGNAL_PAD_WORDS, torch.int32)
    grd.local.normal_()
    val = torch.randn(max_n, device="cuda")
    m, v = torch.zeros_like(val), torch.zeros_like(val)
    shadow = torch.empty(max_n, device="cuda", dtype=torch.bfloat16)
    hyper = torch.zeros(16, device="cuda")
    hyper[:9] = torch.tensor([1e-3, 0.9, 0.999, 1e-8, 0.01, 1.0, 0.9, 0.999, 1.0 / world])
    partials = torch.zeros(256, device="cuda")
    ref = torch.empty(max_n, device="cuda")
    # push form: inbox of 2 x world planes + flags; buckets of up to 4 MB (1024 blocks of 16 KB)
    push_max = min(max_n, 1 << 20)
    pheap = SymmetricHeap(2 * world * push_max * 4 + 2 * world * 1024 * 4 + 8192)
    inbox, pflags = pheap.tensor(2 * world * push_max, torch.float32), pheap.tensor(2 * world * 1024, torch.int32)
    pctl = torch.zeros(4, dtype=torch.int32, device="cuda")
    pout = torch.empty(push_max, device="cuda")
    torch.cuda.synchronize()
    dist.barrier()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def fused(algo, n, adam):
        check(lib.nb_allreduce_fused(
            ctypes.c_int(algo), ctypes.c_int(world), ctypes.c_int(rank), grd.ptr_table(), red.ptr_table(), sig.ptr_table(),
            ctypes.c_void_p(0), ctypes.c_void_p(0), ctypes.c_longlong(n), ptr(val) if adam else None, ptr(m) if adam else None,
            ptr(v) if adam else None, ptr(shadow) if adam else None, None, ptr(hyper) if adam else None, ptr(partials), None,
            ctypes.c_float(0.0), ctypes.c_int(0), ctypes.c_uint(1 << 24), ptr(device_status()), stream_ptr()), "ar")

    def push(n, adam):
        one = lambda t: (ctypes.c_void_p * 1)(t.data_ptr())
        check(lib.nb_allreduce_push(
            ctypes.c_int(world), ctypes.c_int(rank), ctypes.c_int(1), inbox.ptr_table(), pflags.ptr_table(), ptr(pctl),
            one(grd.local), None if adam else one(pout), one(val) if adam else None, one(m) if adam else None,
            one(v) if adam else None, one(shadow) if adam else None, None, one(hyper), (ctypes.c_longlong * 1)(n),
            ctypes.c_int(0), ctypes.c_int(0), ctypes.c_uint(1 << 24), ptr(device_status()), stream_ptr()), "push")

    def nccl(n, adam):
        ref[:n].copy_(grd.local[:n])
        dist.all_reduce(ref[:n])
        if adam:
            check(lib.nb_arena_adamw(ptr(val), ptr(ref), ptr(m), ptr(v), ptr(shadow), None, ctypes.c_longlong(n), ptr(hyper),
                                     ctypes.c_int(0), stream_ptr()), "adamw")

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        ts = []
        for _ in range(args.iters):
            flush.zero_()
            dist.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        ts.sort()
        t = torch.tensor([ts[len(ts) // 2]], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def chained(fn, k=50):
        """k calls back to back inside one event pair: the per-call time inside a captured training step, where the
        ranks' launch skew (tens of microseconds after a host barrier) is paid once, not per call."""
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(k):
            fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / k], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # correctness of the plain all-reduce against NCCL once
    n = 1 << 20
    fused(1, n, False)
    nccl(n, False)
    torch.cuda.synchronize()
    err = (red.local[:n] - ref[:n]).abs().max().item()
    push(n, False)
    torch.cuda.synchronize()
    err = max(err, (pout[:n] * world - ref[:n]).abs().max().item())     # the push form returns the mean (hyper[GSCALE] = 1/N)
    size = 64 << 10
    rows = []
    while size <= args.max_mb << 20:
        n = size // 4
        row = {"bytes": size, "world": world, "adam": args.adam, "check_max_err": err}
        roof_ms = (world - 1) / world * size / (LINK_GBS * 1e9) * 1e3
        for name, algo in (("push", 3), ("one_shot", 0), ("two_shot", 1)):
            if (algo == 0 and size > (16 << 20)) or (algo == 3 and n > push_max):
                continue
            t = timed((lambda: push(n, args.adam)) if algo == 3 else (lambda: fused(algo, n, args.adam)))
            row[name + "_us"] = round(t * 1e3, 2)
            row[name + "_frac_of_roofline"] = round(roof_ms / t, 3)
            row[name + "_frac_of_p2p_bound"] = round(2 * roof_ms / t, 3)
            if size <= (16 << 20):
                row[name + "_chained_us"] = round(chained((lambda: push(n, args.adam)) if algo == 3 else (lambda: fused(algo, n, args.adam))) * 1e3, 2)
        t = timed(lambda: nccl(n, args.adam))
        if size <= (16 << 20):
            row["nccl_chained_us"] = round(chained(lambda: nccl(n, args.adam)) * 1e3, 2)
        row["nccl_us"] = round(t * 1e3, 2)
        row["nccl_frac_of_roofline"] = round(roof_ms / t, 3)
        row["nccl_frac_of_p2p_bound"] = round(2 * roof_ms / t, 3)
        row["busbw_two_shot_gbs"] = round(2 * (world - 1) / world * size / (row["two_shot_us"] * 1e-6) / 1e9, 1)
        rows.append(row)
        if rank == 0 and emit:
            print(json.dumps(row), flush=True)
        size *= 4
    check_status()
    return rows


if __name__ == "__main__":
    main()
