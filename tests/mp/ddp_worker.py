"""Worker of the multi-GPU DDP test: fused P2P all-reduce + Adam vs NCCL all-reduce + local Adam."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from noeira_b200 import nn
    from noeira_b200.ops import check_status
    from noeira_b200.parallel.ddp import FusedGradSync
    ok = True
    for algo, hidden, clip in ((0, 64, 0.0), (1, 256, 0.0), (0, 64, 0.5), (1, 512, 0.5)):
        nn.manual_seed(7)
        net = nn.Sequential(nn.LinearTanh(32, hidden), nn.LinearTanh(hidden, hidden), nn.Linear(hidden, 8)).to("cuda")
        ref = nn.Sequential(nn.LinearTanh(32, hidden), nn.LinearTanh(hidden, hidden), nn.Linear(hidden, 8)).to("cuda")
        ref.copy_from(net)
        opt = nn.AdamW(net.named_params(), lr=1e-2, weight_decay=0.01)
        ropt = nn.AdamW(ref.named_params(), lr=1e-2, weight_decay=0.01)
        opt.max_grad_norm = ropt.max_grad_norm = clip
        sync = FusedGradSync(world, rank, local, algo=algo)
        sync.attach(opt)
        g = torch.Generator(device="cuda").manual_seed(100 + rank)
        for step in range(4):
            x = torch.randn(256, 32, device="cuda", generator=g).bfloat16()
            dy = (torch.randn(256, 8, device="cuda", generator=g) * 0.1).bfloat16()
            for n_, o in ((net, None), (ref, None)):
                n_.forward(x)
                n_.vjp(dy)
            sync.reduce_and_step(opt)
            dist.all_reduce(ropt.arena.grd)
            ropt.hyper[8] = 1.0 / world
            if clip > 0:
                ropt.clip(base_scale=1.0 / world)
            ropt.step(zero_grad=True)
        torch.cuda.synchronize()
        check_status()
        # replicas bit-identical
        mine = opt.arena.val.clone()
        lst = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(lst, mine)
        same = all(torch.equal(lst[0], t) for t in lst)
        err = (opt.arena.val - ropt.arena.val).abs().max().item()
        gz = opt.arena.grd.abs().max().item()
        if rank == 0:
            print(f"algo={algo} hidden={hidden} clip={clip}: replicas_equal={same} max|fused-nccl|={err:.3e} grd_zeroed={gz == 0.0}")
        ok = ok and same and err < (2e-4 if clip > 0 else 2e-5) and gz == 0.0
    ok = push_case(rank, world, local) and ok
    ok = zero_case(rank, world, local) and ok
    ok = overlap_case(rank, world, local) and ok
    dist.barrier()
    if rank == 0:
        print("DDP_WORKER_OK" if ok else "DDP_WORKER_FAIL")
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


def push_case(rank, world, local):
    """Two optimizers reduced and stepped by ONE push kernel (inbox double-buffered by epoch parity, step counters
    advanced in the kernel) against NCCL all-reduce + local Adam, over enough steps to reuse both parities."""
    from noeira_b200 import nn
    from noeira_b200.ops import check_status
    from noeira_b200.parallel.ddp import FusedGradSync
    nn.manual_seed(11)
    mk = lambda o: nn.Sequential(nn.LinearTanh(24, 256), nn.LinearTanh(256, 256), nn.Linear(256, o)).to("cuda")
    nets, refs = [mk(8), mk(1)], [mk(8), mk(1)]
    for n_, r_ in zip(nets, refs):
        r_.copy_from(n_)
    opts = [nn.Adam(n_.named_params(), lr=3e-3) for n_ in nets]
    ropts = [nn.Adam(r_.named_params(), lr=3e-3) for r_ in refs]
    sync = FusedGradSync(world, rank, local)
    sync.attach(*opts)
    assert sync.push is not None
    g = torch.Generator(device="cuda").manual_seed(200 + rank)
    for step in range(5):
        x = torch.randn(512, 24, device="cuda", generator=g).bfloat16()
        for n_, r_, o in zip(nets, refs, (8, 1)):
            dy = (torch.randn(512, o, device="cuda", generator=g) * 0.1).bfloat16()
            for q in (n_, r_):
                q.forward(x)
                q.vjp(dy)
        sync.reduce_and_step_many(opts)
        for ro in ropts:
            dist.all_reduce(ro.arena.grd)
            ro.hyper[8] = 1.0 / world
            ro.step(zero_grad=True)
    torch.cuda.synchronize()
    check_status()
    ok = True
    for o, ro in zip(opts, ropts):
        mine = o.arena.val.clone()
        lst = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(lst, mine)
        same = all(torch.equal(lst[0], t) for t in lst)
        err = (o.arena.val - ro.arena.val).abs().max().item()
        steps_equal = torch.equal(o.hyper[5:8], ro.hyper[5:8])
        gz = o.arena.grd.abs().max().item()
        if rank == 0:
            print(f"push numel={o.arena.numel}: replicas_equal={same} max|fused-nccl|={err:.3e} step_counters_equal={steps_equal} "
                  f"grd_zeroed={gz == 0.0}")
        ok = ok and same and err < 2e-5 and steps_equal and gz == 0.0
    # plain sum through the same kernel
    one = nn.Adam(mk(2).named_params(), lr=1e-3)
    s2 = FusedGradSync(world, rank, local)
    s2.attach(one)
    one.arena.grd.copy_(torch.full_like(one.arena.grd, float(rank + 1)))
    red = s2.all_reduce(one)
    torch.cuda.synchronize()
    want = sum(range(1, world + 1)) / world
    okp = bool((red - want).abs().max().item() < 1e-6)
    if rank == 0:
        print(f"push plain all-reduce: ok={okp}")
    return ok and okp


def zero_case(rank, world, local):
    """Fused ZeRO-1 step (reduce-scatter + shard AdamW + all-gather with bf16 recast in one kernel) against NCCL
    all-reduce + the full local AdamW: same values, identical replicas, moments only at shard size."""
    from noeira_b200 import nn
    from noeira_b200.ops import check_status
    from noeira_b200.parallel.ddp import FusedZeroSync
    nn.manual_seed(21)
    mk = lambda: nn.Sequential(nn.LinearTanh(32, 384), nn.LinearTanh(384, 384), nn.Linear(384, 8)).to("cuda")
    net, ref = mk(), mk()
    ref.copy_from(net)
    opt = nn.AdamW(net.named_params(), lr=1e-2, weight_decay=0.01)
    ropt = nn.AdamW(ref.named_params(), lr=1e-2, weight_decay=0.01)
    full_moment_bytes = opt.arena.m.numel() * 4
    sync = FusedZeroSync(world, rank, local)
    sync.attach(opt)
    g = torch.Generator(device="cuda").manual_seed(300 + rank)
    for step in range(4):
        x = torch.randn(256, 32, device="cuda", generator=g).bfloat16()
        dy = (torch.randn(256, 8, device="cuda", generator=g) * 0.1).bfloat16()
        for q in (net, ref):
            q.forward(x)
            q.vjp(dy)
        sync.reduce_and_step(opt)
        dist.all_reduce(ropt.arena.grd)
        ropt.hyper[8] = 1.0 / world
        ropt.step(zero_grad=True)
    torch.cuda.synchronize()
    check_status()
    mine = opt.arena.val.clone()
    lst = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(lst, mine)
    same = all(torch.equal(lst[0], t) for t in lst)
    err = (opt.arena.val - ropt.arena.val).abs().max().item()
    sherr = (opt.arena.shadow.float() - opt.arena.val).abs().max().item()
    shard_ok = sync.state[id(opt)]["m"].numel() * 4 <= full_moment_bytes / world + 4096
    gz = opt.arena.grd.abs().max().item()
    if rank == 0:
        print(f"zero numel={opt.arena.numel}: replicas_equal={same} max|fused-nccl|={err:.3e} shadow_err={sherr:.2e} "
              f"moments_sharded={shard_ok} grd_zeroed={gz == 0.0}")
    # lr = 1e-2: the library's ring order and this kernel's rank order sum the gradients differently, and Adam turns
    # a last-bit difference of a near-zero gradient into a difference of a fraction of lr
    return same and err < 2e-4 and sherr < 2e-2 and shard_ok and gz == 0.0


def overlap_case(rank, world, local):
    """A small GPT trained by the autoregressive trainer with the gradient reduction overlapped with the backward
    (bucketed NCCL all-reduces launched from the units' vjp) against the reduce-after-backward NCCL baseline: identical
    replicas, matching losses, and buckets that really left during the backward."""
    from noeira_b200.models.gpt import GPT
    from noeira_b200.ops import check_status
    from noeira_b200.parallel.ddp import NcclGradSync, OverlapGradSync
    from noeira_b200.training.trainer import AutoregressiveTrainer
    torch.manual_seed(3)
    tokens = torch.randint(0, 96, (20000,), device="cuda")
    losses, vals, during = [], [], 0
    for kind in ("overlap", "nccl"):
        model = GPT(vocab=96, seq=64, dim=128, layers=3, heads=2, seed=5).to("cuda")
        sync = OverlapGradSync(world, rank, bucket_bytes=256 << 10) if kind == "overlap" else NcclGradSync(world, rank)
        tr = AutoregressiveTrainer(model, tokens, batch=8, seq=64, lr=1e-3, warmup=2, total_steps=20, seed=9, grad_sync=sync,
                                   rank=rank, world=world)
        ls = [float(tr.train_step()) for _ in range(6)]
        torch.cuda.synchronize()
        check_status()
        losses.append(ls)
        vals.append(tr.opt.arena.val.clone())
        if kind == "overlap":
            during, nb = sync.st.launched_during_backward, len(sync.st.buckets)
    mine = vals[0]
    lst = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(lst, mine)
    same = all(torch.equal(lst[0], t) for t in lst)
    err = (vals[0] - vals[1]).abs().max().item()
    dl = max(abs(a - b) for a, b in zip(*losses))
    if rank == 0:
        print(f"overlap: buckets={nb} launched_during_backward={during} replicas_equal={same} max|overlap-nccl|={err:.3e} "
              f"max loss diff={dl:.3e}")
    # the bucketed and the whole-arena reductions sum the ranks in different orders; Adam turns a last-bit difference of a
    # near-zero gradient into a step of up to lr, so after 6 steps at lr = 1e-3 single elements may differ by a few lr
    # (measured 2.9e-3 at 8 ranks), while the losses agree to 1e-4
    return same and nb >= 3 and during >= 6 * (nb - 1) and err < 8e-3 and dl < 5e-3


if __name__ == "__main__":
    try:
        main()
    except Exception:                      # the launcher keeps only the tail of stderr: put the traceback on stdout too
        import traceback
        print(f"rank {os.environ.get('RANK')} raised:\n{traceback.format_exc()}", flush=True)
        raise
