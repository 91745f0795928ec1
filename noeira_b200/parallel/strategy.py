"""Sharding strategies over the parameter arena: DDP, ZeRO-1, ZeRO-2, ZeRO-3 (FSDP FULL_SHARD).

All strategies share one interface (the reference's ``ShardingStrategy`` trait,
noeira/nn/distributed/strategy.mojo:45-124): ``sync_params``, ``reduce_grads``, ``clip_grads``, ``step``,
``state_bytes_per_rank``; they operate on the flat arena of an optimizer, so no per-module hooks are needed:

  DataParallel   all-reduce the gradient arena, every rank runs the full optimizer                (5Ψ bytes/elem·4)
  Zero1          reduce-scatter gradients, each rank updates its shard (rows of the arena), all-gather values
  Zero2          like ZeRO-1 but the full gradient arena is released after the reduce-scatter (shard only kept)
  Zero3          values are sharded too: ``gather_params`` before forward/backward, ``release_params`` after

Shards are contiguous ranges of the arena rounded to PARAM_ALIGN rows (noeira/nn/distributed/zero.mojo:18-22;
``shard_rows`` process_group.mojo:63-74).  Reductions go through a ``Comm`` (ThreadComm simulator, gloo, nccl), so
DDP and ZeRO are bit-identical without clipping, as the reference gates require.  On GPUs the DDP path is
replaced by the fused all-reduce+Adam kernel (``parallel.ddp.FusedGradSync``).
"""
from __future__ import annotations

import math

import torch

from ..nn.arena import PARAM_ALIGN
from ..nn.optim import H_B1T, H_B2T, H_BETA1, H_BETA2, H_EPS, H_GSCALE, H_LR, H_T, H_WD, Optimizer, adamw_update_cpu


def shard_range(numel: int, world: int, rank: int):
    rows = numel // PARAM_ALIGN
    per = (rows + world - 1) // world
    lo = min(rows, per * rank) * PARAM_ALIGN
    hi = min(rows, per * (rank + 1)) * PARAM_ALIGN
    return lo, hi, per * PARAM_ALIGN


class DataParallel:
    name = "ddp"

    def __init__(self, opt: Optimizer, comm):
        self.opt, self.comm = opt, comm
        self.world, self.rank = comm.world, comm.rank

    def sync_params(self):
        self.comm.broadcast(self.opt.arena.val, 0)
        if self.opt.arena.shadow is not None:
            self.opt.arena.refresh_shadow()

    def reduce_grads(self):
        self.comm.all_reduce(self.opt.arena.grd)
        self.opt.arena.grd.mul_(1.0 / self.world)

    def grad_norm(self):
        return float(self.opt.arena.grd.double().pow(2).sum().sqrt())

    def clip_grads(self, max_norm):
        n = self.grad_norm()
        s = 0.0 if not math.isfinite(n) else (max_norm / (n + 1e-6) if n > max_norm > 0 else 1.0)
        self.opt.arena.grd.mul_(s)
        return n

    def step(self):
        self.opt.step(zero_grad=True)

    def state_bytes_per_rank(self):
        return self.opt.arena.numel * 4 * 4  # val, grd, m, v


class Zero1(DataParallel):
    name = "zero1"

    def __init__(self, opt, comm):
        super().__init__(opt, comm)
        a = opt.arena
        self.lo, self.hi, self.per = shard_range(a.numel, self.world, self.rank)
        self.padded = self.per * self.world
        self._gpad = torch.zeros(self.padded, dtype=torch.float32, device=a.val.device)
        self._gshard = torch.zeros(self.per, dtype=torch.float32, device=a.val.device)
        self._vpad = torch.zeros(self.padded, dtype=torch.float32, device=a.val.device)

    def reduce_grads(self):
        a = self.opt.arena
        self._gpad[: a.numel].copy_(a.grd)
        self.comm.reduce_scatter(self._gshard, self._gpad)
        self._gshard.mul_(1.0 / self.world)

    def grad_norm(self):
        ss = self._gshard[: self.hi - self.lo].double().pow(2).sum().reshape(1).float()
        t = ss.clone()
        self.comm.all_reduce(t)
        return float(t.sqrt())

    def clip_grads(self, max_norm):
        n = self.grad_norm()
        s = 0.0 if not math.isfinite(n) else (max_norm / (n + 1e-6) if n > max_norm > 0 else 1.0)
        self._gshard.mul_(s)
        return n

    def _adam_shard(self):
        """AdamW on [lo, hi) with exactly the arithmetic of the arena kernel / CPU optimizer."""
        a, h = self.opt.arena, self.opt.hyper
        h[H_T] += 1
        h[H_B1T] *= h[H_BETA1]
        h[H_B2T] *= h[H_BETA2]
        lr, b1, b2, eps, wd, b1t, b2t, gs = (float(h[i]) for i in (H_LR, H_BETA1, H_BETA2, H_EPS, H_WD, H_B1T, H_B2T, H_GSCALE))
        lo, hi = self.lo, self.hi
        n = hi - lo
        if n <= 0:
            return
        flags = a.row_flags.repeat_interleave(PARAM_ALIGN)[lo:hi]
        g = self._gshard[:n] if gs == 1.0 else self._gshard[:n] * gs
        adamw_update_cpu(a.val[lo:hi], g, a.m[lo:hi], a.v[lo:hi], flags, lr, b1, b2, eps, wd, b1t, b2t)

    def step(self):
        a = self.opt.arena
        self._adam_shard()
        shard = torch.zeros(self.per, dtype=torch.float32, device=a.val.device)
        shard[: self.hi - self.lo] = a.val[self.lo:self.hi]
        self.comm.all_gather(self._vpad, shard)
        a.val.copy_(self._vpad[: a.numel])
        a.grd.zero_()
        a.bump_versions(shadow_fresh=False)
        if a.shadow is not None:
            a.refresh_shadow()

    def state_bytes_per_rank(self):
        n = self.opt.arena.numel
        return n * 4 * 2 + self.per * 4 * 3  # val + grd full, m/v/grad shard


class Zero2(Zero1):
    """Gradient arena is not retained between steps beyond the local shard (2Ψ → Ψ + Ψ/N for grads)."""
    name = "zero2"

    def state_bytes_per_rank(self):
        n = self.opt.arena.numel
        return n * 4 + self.per * 4 * 3


class Zero3(Zero1):
    """Values are sharded between steps; ``gather_params`` materialises them for forward/backward."""
    name = "zero3"

    def __init__(self, opt, comm):
        super().__init__(opt, comm)
        self.gathered = True

    def release_params(self):
        a = self.opt.arena
        keep = a.val[self.lo:self.hi].clone()
        a.val.zero_()
        a.val[self.lo:self.hi] = keep
        self.gathered = False

    def gather_params(self):
        a = self.opt.arena
        shard = torch.zeros(self.per, dtype=torch.float32, device=a.val.device)
        shard[: self.hi - self.lo] = a.val[self.lo:self.hi]
        self.comm.all_gather(self._vpad, shard)
        a.val.copy_(self._vpad[: a.numel])
        a.bump_versions(shadow_fresh=False)
        self.gathered = True

    def step(self):
        super().step()
        self.release_params()

    def state_bytes_per_rank(self):
        return self.per * 4 * 4


STRATEGIES = {"ddp": DataParallel, "zero1": Zero1, "zero2": Zero2, "zero3": Zero3}
