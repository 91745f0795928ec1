"""Secondary benchmark workloads behind ``bench.py --workload {act,vla,wm,sac_cpu,secondary}``.

wm   Dreamer-style world-model dynamics transformer (24 × d2048, 16/4 heads GQA, SwiGLU 5632, block-causal over
     64 frames × (256 latents + 1 action token)), flow-matching loss, AdamW 3e-4, bf16, tensor parallel over all N
     ranks with sequence-parallel activations (fused all-gather→GEMM and GEMM→reduce-scatter kernels).
     Global batch = one sequence per rank (8 at N = 8).  Metric: sequences / s.
"""
import json
import time

import torch
import torch.distributed as dist


def run(args, rank, local_rank, world):
    try:
        return _run(args, rank, local_rank, world)
    except Exception:  # noqa: BLE001 — a launcher keeps only its own traceback; print the worker's cause on stdout
        import traceback
        print(json.dumps({"workload": args.workload, "rank": rank, "error": traceback.format_exc()[-1500:]}), flush=True)
        raise


def run_secondary(args, rank, local_rank, world):
    """ACT, VLA, world model (tensor parallel over all ranks) and the all-reduce table, one after the other in this
    process group; each prints its own JSON line, a failure of one is reported and the next one still runs."""
    import copy
    import gc
    plan = (("act", 5), ("vla", 3), ("wm", 2), ("allreduce", 5))
    for name, steps in plan:
        a = copy.copy(args)
        a.workload, a.steps, a.warmup = name, steps, 3
        try:
            if name == "wm":
                run_wm(a, rank, local_rank, world, finalize=False)
            elif name == "allreduce":
                if world > 1:
                    run_allreduce(a, rank, local_rank, world)
            else:
                run_dp(a, rank, local_rank, world, finalize=False)
        except Exception:  # noqa: BLE001
            import traceback
            if rank == 0:
                print(json.dumps({"workload": name, "error": traceback.format_exc()[-800:]}), flush=True)
        gc.collect()
        torch.cuda.empty_cache()
        if world > 1:
            dist.barrier()
    if world > 1:
        dist.destroy_process_group()
    return 0


def run_allreduce(args, rank, local_rank, world):
    """Fused all-reduce forms against NCCL at a few bucket sizes (the full table: benchmarks/bench_allreduce.py)."""
    from benchmarks import bench_allreduce
    rows = bench_allreduce.table(rank, world, max_mb=64, iters=5, adam=False, emit=False)
    if rank == 0:
        print(json.dumps({"metric": "allreduce_us", "n_gpus": world, "unit": "us", "rows": rows}), flush=True)


def _run(args, rank, local_rank, world):
    if args.workload == "secondary":
        return run_secondary(args, rank, local_rank, world)
    if args.workload == "wm":
        return run_wm(args, rank, local_rank, world)
    if args.workload in ("act", "vla"):
        return run_dp(args, rank, local_rank, world)
    if args.workload == "sac_cpu":
        return run_sac_cpu(args)
    raise SystemExit(f"unknown workload {args.workload}")


def run_wm(args, rank, local_rank, world, finalize=True):
    from noeira_b200 import _native
    from noeira_b200.models.world_model import WorldModel, WorldModelConfig
    from noeira_b200.ops import check_status
    from noeira_b200.parallel.ddp import FusedGradSync
    from noeira_b200.utils.bench_utils import timed_steps
    cfg = WorldModelConfig()
    if getattr(args, "small", False):
        cfg = WorldModelConfig(layers=4, dim=1024, heads=8, kv_heads=1, ff=2816, frames=16)
    B = world  # one sequence per rank
    sync = FusedGradSync(world, rank, local_rank) if world > 1 else None
    model = WorldModel(cfg, batch=B, world=world, rank=rank, grad_sync=sync)
    ms = model.ms
    # synthetic data staged in pinned host memory; every step copies this rank's shard to the device
    z1_h = (torch.randn(ms, cfg.latent_dim)).pin_memory()
    act_h = (torch.rand(ms, cfg.action_dim) * 2 - 1).pin_memory()
    z1 = torch.empty(ms, cfg.latent_dim, device="cuda")
    act = torch.empty(ms, cfg.action_dim, device="cuda")
    loss_h = torch.zeros(1).pin_memory()
    gen = torch.Generator(device="cuda").manual_seed(1 + rank)
    tgen = torch.Generator(device="cuda").manual_seed(7)   # same flow times on every rank
    rows_seq = torch.arange(ms, device="cuda") // model.S + (rank * ms) // model.S

    def step(e2e=False):
        if e2e:
            z1.copy_(z1_h, non_blocking=True)
            act.copy_(act_h, non_blocking=True)
        noise = torch.randn(ms, cfg.latent_dim, device="cuda", generator=gen)
        t = torch.rand(B, device="cuda", generator=tgen)[rows_seq]
        model.loss_acc.zero_()
        model.train_step(z1 * model.is_lat[:, None], act, noise * model.is_lat[:, None], t)
        if e2e:
            loss_h.copy_(model.loss_acc, non_blocking=True)
            torch.cuda.synchronize()

    z1.copy_(z1_h)
    act.copy_(act_h)
    n0 = _native.launch_count()
    total_ms, clocks = timed_steps(step, args.steps, args.warmup, world, rank, local_rank)
    launches = (_native.launch_count() - n0) * args.steps // (args.steps + max(args.warmup, 3))
    check_status()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step(e2e=True)
    if world > 1:
        dist.barrier()
    e2e_s = time.perf_counter() - t0
    tt = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    e2e_s = float(tt.item())
    loss = float(model.loss_acc.item())
    # model FLOPs per sequence: 6 · params · tokens + attention (block-causal ≈ half of S²)
    S = cfg.seq_len
    flops = 6.0 * cfg.num_params() * S + 3 * 4.0 * cfg.layers * cfg.heads * cfg.head_dim * S * S * 0.5 * (1 + cfg.frame_len / S)
    if rank == 0:
        sps = B * args.steps / (total_ms / 1e3)
        print(json.dumps({
            "metric": "world_model_train_sequences_per_s", "value": round(sps, 4), "unit": "sequences/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(total_ms / args.steps, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (latents ~N(0,1)^32, actions ~U(-1,1)^6, random-init weights)",
            "config": {"model": f"dynamics transformer {cfg.layers}x{cfg.dim}, {cfg.heads}/{cfg.kv_heads} heads, ff {cfg.ff}, "
                                f"{cfg.num_params() / 1e9:.2f}B params", "global_batch": B, "seq_len": S,
                       "parallelism": f"tp{world}+sp", "l2": "flushed between timed iterations"},
            "model_tflops_per_gpu": round(flops * sps / world / 1e12, 1),
            "clocks": clocks,
            "e2e": {"value": round(B * args.steps / e2e_s, 4), "unit": "sequences/s",
                    "h2d_bytes_per_step": int(z1_h.numel() * 4 + act_h.numel() * 4), "d2h_bytes_per_step": 4},
            "gpu_launches": launches, "final_loss": round(loss, 5)}))
    if world > 1 and finalize:
        dist.destroy_process_group()
    return 0


def run_dp(args, rank, local_rank, world, finalize=True):
    """ACT (batch 8 / GPU, 2 cameras 3x480x640 uint8) and SmolVLA-style VLA (batch 64 / GPU, 3 cameras 3x512x512),
    data parallel with the fused gradient all-reduce + AdamW kernel.  Metric: training samples / s (whole job)."""
    from noeira_b200 import _native
    from noeira_b200.ops import check_status
    from noeira_b200.parallel.ddp import FusedGradSync
    from noeira_b200.utils.bench_utils import timed_steps
    sync = FusedGradSync(world, rank, local_rank) if world > 1 else None
    g = torch.Generator().manual_seed(100 + rank)
    if args.workload == "act":
        from noeira_b200.models.act import ACTConfig, ACTTrainer
        cfg = ACTConfig()
        B = 8
        if args.small:
            cfg = ACTConfig(height=96, width=128, chunk=20, enc_layers=1, dec_layers=1)
        tr = ACTTrainer(cfg, grad_sync=sync)
        host = dict(qpos=torch.randn(B, 6, generator=g).pin_memory(),
                    img=torch.randint(0, 256, (B, cfg.n_cam, 3, cfg.height, cfg.width), dtype=torch.uint8, generator=g).pin_memory(),
                    act=torch.randn(B, cfg.chunk, 6, generator=g).pin_memory())
        dev = {k: v.cuda() for k, v in host.items()}
        valid = torch.ones(B, cfg.chunk + 2, device="cuda")
        step_fn = lambda: (tr.train_step if args.eager else tr.step)(dev["qpos"], dev["img"], dev["act"], valid)
        model_desc = f"ACT ResNet-18 + DETR enc {cfg.enc_layers}/dec {cfg.dec_layers}, d {cfg.dim}, chunk {cfg.chunk}, {cfg.n_cam} cams {cfg.height}x{cfg.width}"
        loss_of = lambda: float(tr.loss_acc[0])
    else:
        from noeira_b200.models.vla import VLAConfig, VLATrainer
        cfg = VLAConfig()
        B = 64
        if args.small:
            cfg = VLAConfig(image=128, vit_layers=2, lm_layers=2)
            B = 8
        tr = VLATrainer(cfg, grad_sync=sync)
        host = dict(img=torch.rand(B, cfg.n_cam, 3, cfg.image, cfg.image, generator=g).to(torch.bfloat16).pin_memory(),
                    ids=torch.randint(0, cfg.vocab, (B, cfg.n_lang), generator=g).pin_memory(),
                    state=torch.randn(B, cfg.action_dim, generator=g).pin_memory(),
                    act=torch.randn(B, cfg.chunk, cfg.action_dim, generator=g).pin_memory())
        dev = {k: v.cuda() for k, v in host.items()}
        step_fn = lambda: (tr.train_step if args.eager else tr.step)(dev["img"], dev["ids"], dev["state"], dev["act"])
        model_desc = (f"ViT {cfg.vit_layers}x{cfg.vit_dim} + LM {cfg.lm_layers}x{cfg.hidden} ({cfg.heads}/{cfg.kv_heads} heads) + "
                      f"expert {cfg.lm_layers}x{cfg.expert_width}, {cfg.n_cam} cams {cfg.image}^2, chunk {cfg.chunk}; prefix frozen")
        loss_of = lambda: float(tr.loss_acc[0])

    def e2e_step():
        for k in host:
            dev[k].copy_(host[k], non_blocking=True)
        step_fn()
        _ = loss_of()

    n0 = _native.launch_count()
    total_ms, clocks = timed_steps(step_fn, args.steps, args.warmup, world, rank, local_rank)
    launches = (_native.launch_count() - n0) * args.steps // (args.steps + max(args.warmup, 3))
    check_status()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    if world > 1:
        dist.barrier()
    e2e_s = time.perf_counter() - t0
    tt = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    e2e_s = float(tt.item())
    if rank == 0:
        sps = B * world * args.steps / (total_ms / 1e3)
        print(json.dumps({
            "metric": f"{args.workload}_train_samples_per_s", "value": round(sps, 2), "unit": "samples/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(total_ms / args.steps, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (seed-generated inputs, random-init weights)",
            "config": {"model": model_desc, "global_batch": B * world, "seq_len": cfg.chunk, "parallelism": f"dp{world}",
                       "l2": "flushed between timed iterations"},
            "clocks": clocks,
            "e2e": {"value": round(B * world * args.steps / e2e_s, 2), "unit": "samples/s",
                    "h2d_bytes_per_step": int(sum(v.numel() * v.element_size() for v in host.values())), "d2h_bytes_per_step": 4},
            "gpu_launches": launches, "params_m": round(sum(p.numel for _, p in tr.model.named_params()) / 1e6, 1),
            "final_loss": round(loss_of(), 5)}))
    if world > 1 and finalize:
        dist.destroy_process_group()
    return 0


def run_sac_cpu(args):
    """SAC update on the CPU in fp32 (actor 17-256-256-(6+6) tanh-Gaussian, twin critics 23-256-256-1 with targets,
    batch 256 of seed-generated transitions, Adam 3e-4, tau 0.005, gamma 0.99, automatic entropy): updates per second
    through the explicit-backward ``nn`` path (this is the numerics-oracle path of the framework; no GPU involved)."""
    from noeira_b200.agents.sac import SACConfig, SACTrainer
    torch.manual_seed(0)
    cfg = SACConfig()
    tr = SACTrainer(cfg, device="cpu")
    g = torch.Generator().manual_seed(0)
    B = cfg.batch
    s, sp = torch.randn(B, 17, generator=g), torch.randn(B, 17, generator=g)
    a = torch.rand(B, 6, generator=g) * 2 - 1
    r = torch.randn(B, generator=g)
    d = (torch.rand(B, generator=g) < 0.01).float()
    for _ in range(max(args.warmup, 3)):
        tr.update(s, a, r, sp, d)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        m = tr.update(s, a, r, sp, d)
    dt = time.perf_counter() - t0
    print(json.dumps({"metric": "sac_cpu_updates_per_s", "value": round(args.steps / dt, 2), "unit": "updates/s", "n_gpus": 0,
                      "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(dt / args.steps * 1e3, 3),
                      "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32",
                      "data": "synthetic (seed-generated transitions, random-init weights)",
                      "config": {"model": "SAC actor 17-256-256-12, twin critics 23-256-256-1 + targets", "global_batch": B,
                                 "seq_len": 1, "parallelism": "cpu", "threads": torch.get_num_threads()},
                      "gpu_launches": 0, "metrics": {k: (round(float(v), 5) if v == v else None) for k, v in (m or {}).items()} if isinstance(m, dict) else None}))
    return 0
