"""Worker of the tensor-parallel test: fused AG→GEMM / GEMM→RS kernels vs NCCL + unfused GEMM."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from noeira_b200.ops import check_status
    from noeira_b200.parallel.tp import NcclTP, TPLinearContext
    ok = True
    base = NcclTP(world, rank)
    for (ms, k, n, b_mn) in ((256, 512, 384, True), (128, 2048, 256, False), (384, 320, 1408, True)):
        g = torch.Generator(device="cuda").manual_seed(10 + rank)
        gw = torch.Generator(device="cuda").manual_seed(99)
        # ---- all-gather → GEMM (column parallel)
        ctx = TPLinearContext(world, rank, ms, k, n, "ag")
        w = (torch.randn((k, n) if b_mn else (n, k), device="cuda", generator=gw) * 0.05).bfloat16()
        bias = torch.randn(n, device="cuda", generator=gw)
        for it in range(3):
            x = (torch.randn(ms, k, device="cuda", generator=g)).bfloat16()
            ctx.x_shard.copy_(x)
            y = ctx.ag_gemm(w, b_mn, bias=bias, act="gelu")
            ref, full = base.ag_gemm(x, w, b_mn, bias=bias, act="gelu")
            torch.cuda.synchronize()
            e1 = (y.float() - ref.float()).abs().max().item()
            e2 = (ctx.gathered_input().float() - full.float()).abs().max().item()
            ok = ok and e1 < 2e-2 * max(1.0, ref.float().abs().max().item()) and e2 == 0.0
            if rank == 0:
                print(f"ag_gemm ms={ms} k={k} n={n} b_mn={b_mn} it={it}: max|fused-nccl|={e1:.3e} gather_err={e2:.1e}")
        # ---- GEMM → reduce-scatter (row parallel): a [P·ms, k] local, out [ms, n]
        ctx2 = TPLinearContext(world, rank, ms, k, n - n % 8, "rs")
        n2 = n - n % 8
        w2 = (torch.randn((k, n2) if b_mn else (n2, k), device="cuda", generator=gw) * 0.05).bfloat16()
        for it in range(3):
            a = torch.randn(world * ms, k, device="cuda", generator=g).bfloat16()
            res = torch.randn(ms, n2, device="cuda", generator=g).bfloat16()
            out = ctx2.gemm_rs(a, w2, b_mn, residual=res)
            ref = base.gemm_rs(a, w2, b_mn, residual=res)
            torch.cuda.synchronize()
            e = (out.float() - ref.float()).abs().max().item()
            tol = 4e-2 * max(1.0, ref.float().abs().max().item())
            ok = ok and e < tol
            if it == 2:
                again = ctx2.gemm_rs(a, w2, b_mn, residual=res)
                torch.cuda.synchronize()
                ok = ok and torch.equal(out, again)            # slot sums run in rank order: the same bits every time
            if rank == 0:
                print(f"gemm_rs ms={ms} k={k} n={n2} b_mn={b_mn} it={it}: max|fused-nccl|={e:.3e}")
        check_status()
    if world > 1:
        t = torch.tensor([1.0 if ok else 0.0], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        ok = bool(t.item() > 0.5)
        dist.barrier()
    if rank == 0:
        print("TP_WORKER_OK" if ok else "TP_WORKER_FAIL")
    if world > 1:
        dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
