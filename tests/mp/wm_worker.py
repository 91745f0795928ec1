"""Worker of the tensor-parallel world-model test: the TP + SP model on P ranks against the same model on one rank
(same seed → the same full weight matrices, every rank keeps its slice), four optimisation steps on one batch."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from noeira_b200.models.world_model import WorldModel, WorldModelConfig
    from noeira_b200.ops import check_status
    from noeira_b200.parallel.ddp import FusedGradSync
    cfg = WorldModelConfig(layers=2, dim=256, heads=8, kv_heads=2, head_dim=64, ff=1024, frames=4, tokens_per_frame=31,
                           latent_dim=32, action_dim=6, lr=1e-3)
    B = world
    tp = WorldModel(cfg, batch=B, world=world, rank=rank, grad_sync=FusedGradSync(world, rank, local))
    ref = WorldModel(cfg, batch=B, world=1, rank=0)
    S = tp.S
    g = torch.Generator(device="cuda").manual_seed(0)
    rows = B * S
    z1 = torch.randn(rows, 32, device="cuda", generator=g)
    nz = torch.randn(rows, 32, device="cuda", generator=g)
    act = torch.rand(rows, 6, device="cuda", generator=g) * 2 - 1
    t = torch.rand(B, device="cuda", generator=g).repeat_interleave(S)
    lo, hi = rank * tp.ms, (rank + 1) * tp.ms
    ok = True
    for step in range(4):
        ref.loss_acc.zero_()
        ref.train_step(z1 * ref.is_lat[:, None], act, nz * ref.is_lat[:, None], t)
        tp.loss_acc.zero_()
        tp.train_step(z1[lo:hi] * tp.is_lat[:, None], act[lo:hi], nz[lo:hi] * tp.is_lat[:, None], t[lo:hi])
        torch.cuda.synchronize()
        check_status()
        total = tp.loss_acc.clone()
        dist.all_reduce(total)
        a, b = float(total), float(ref.loss_acc)
        if rank == 0:
            print(f"step {step}: loss tp{world}+sp = {a:.5f}   one rank = {b:.5f}")
        ok = ok and abs(a - b) < 3e-2 * max(abs(b), 1e-3)
        if step == 0:
            first = b
    ok = ok and b < first            # the shared trajectory goes down
    flag = torch.tensor([1.0 if ok else 0.0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    ok = bool(flag.item() > 0.5)
    dist.barrier()
    if rank == 0:
        print("WM_WORKER_OK" if ok else "WM_WORKER_FAIL")
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
