"""gloo rank of tests/test_elastic_cpu.py: data-parallel training with a heartbeat; in phase 1 the last rank leaves
between steps after the checkpoint, the others notice BEFORE their next collective and stop; phase 2 resumes the
checkpoint under the smaller world size."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def build():
    from noeira_b200 import nn
    nn.manual_seed(5)
    net = nn.Sequential(nn.LinearTanh(12, 40), nn.LinearTanh(40, 40), nn.Linear(40, 3))
    return net, nn.AdamW(net.named_params(), lr=1e-2, weight_decay=0.01)


def batch(step, gb=12):
    g = torch.Generator().manual_seed(1000 + step)
    return torch.randn(gb, 12, generator=g), torch.randn(gb, 3, generator=g)


def main():
    from noeira_b200.io.checkpoint import load_checkpoint, save_checkpoint
    from noeira_b200.parallel.elastic import Heartbeat, PeerLost, resume_plan
    from noeira_b200.parallel.fibers import DistComm
    from noeira_b200.parallel.strategy import DataParallel
    phase, out, ckpt = os.environ["PHASE"], os.environ["OUT"], os.environ["CKPT"]
    total, leave_at = int(os.environ["TOTAL_STEPS"]), int(os.environ.get("LEAVE_AT", "-1"))
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, deadline_s=20.0, prefix="hb" + phase)
    net, opt = build()
    start = 0
    if phase == "2":
        sc = load_checkpoint(ckpt, list(net.named_params()), [])
        opt.load_scalars({k.split(".", 1)[1]: v for k, v in sc.items() if k.startswith("opt.")})
        start = int(sc["step"])
    st = DataParallel(opt, DistComm())
    if phase == "1":
        st.sync_params()
    status = "done"
    for step in range(start, total):
        try:
            hb.check()                                   # before any collective of this step
        except PeerLost as e:
            status = f"peer_lost:{e.ranks}:{step}"
            break
        x, y = batch(step)
        lo, hi = resume_plan(x.shape[0], world, rank)
        o = net.forward(x[lo:hi])
        net.vjp(2.0 * (o - y[lo:hi]) / (hi - lo))
        st.reduce_grads()
        st.step()
        if phase == "1" and step + 1 == leave_at:
            # everyone checkpoints the same state; the store is the rendezvous that orders "checkpoint written"
            # before "rank left"
            if rank == 0:
                save_checkpoint(ckpt, list(net.named_params()), [], {"step": float(step + 1),
                                **{f"opt.{k}": v for k, v in opt.scalars().items()}}, with_moments=True)
            dist.barrier()
            if rank == world - 1:
                hb.leave()
                status = "left"
                break
            # survivors: give the departure a moment to be published, then go on to the next step's check
            import time
            for _ in range(200):
                if hb.peers()[world - 1][1] is None:
                    break
                time.sleep(0.01)
        hb.beat()
    torch.save({"status": status, "val": opt.arena.val.clone()}, f"{out}.p{phase}.r{rank}")
    # no destroy_process_group: after a departure a collective shutdown would wait for the rank that left


if __name__ == "__main__":
    main()
