"""Sharding strategies over the parameter arena: DDP, ZeRO-1, ZeRO-2, ZeRO-3 (FSDP FULL_SHARD).

All strategies share one interface (the reference's ``ShardingStrategy`` trait,
noeira/nn/distributed/strategy.mojo:45-124): ``sync_params``, ``begin_step``, ``reduce_grads``, ``clip_grads``,
``step``, ``state_bytes_per_rank``; they operate on the flat arena of an optimizer:

  DataParallel   all-reduce the gradient arena, every rank runs the full optimizer (val, grd, m, v: 4Ψ floats)
  Zero1          Adam moments exist ONLY as a shard per rank; gradients are reduce-scattered into a shard-size buffer,
                 the rank updates its shard of the values in place and the values are all-gathered in place
                 (2Ψ + 3Ψ/N floats; noeira/nn/distributed/zero.mojo:284-402)
  Zero2          as ZeRO-1, and the full gradient arena is RELEASED after the reduce-scatter (its storage is shrunk to
                 zero and re-materialised by ``begin_step`` before the next backward): Ψ + 3Ψ/N floats between steps
  Zero3          values are sharded too, per UNIT (a top-level block of the model): a unit's values are all-gathered
                 right before its forward and again before its backward and released right after; its gradients are
                 reduce-scattered and released right after its backward (PRE_FORWARD / PRE_VJP / POST_VJP hooks of
                 noeira/nn/distributed/zero_sharded.mojo:249-274, 577-616): 4Ψ/N floats between steps, plus one
                 unit's values and gradients while that unit runs

Shards are contiguous ranges rounded to PARAM_ALIGN rows (noeira/nn/distributed/zero.mojo:18-22; ``shard_rows``
process_group.mojo:63-74).  Releasing memory uses ``untyped_storage().resize_``: every parameter keeps its view, the
bytes go back to the allocator.  Reductions go through a ``Comm`` (ThreadComm simulator, gloo, nccl) whose sums are
rank-ordered, so DDP and ZeRO are bit-identical without clipping, as the reference's gates require.  On GPUs the
DDP path is replaced by the fused all-reduce + Adam kernel (``parallel.ddp.FusedGradSync``) and the ZeRO-1 step by the
fused reduce-scatter + shard-Adam + all-gather kernel (``parallel.ddp.FusedZeroSync``).
"""
from __future__ import annotations

import math
from typing import List

import torch

from ..nn.arena import PARAM_ALIGN
from ..nn.optim import H_B1T, H_B2T, H_BETA1, H_BETA2, H_EPS, H_GSCALE, H_LR, H_T, H_WD, Optimizer, adamw_update_cpu


def shard_range(numel: int, world: int, rank: int):
    rows = numel // PARAM_ALIGN
    per = (rows + world - 1) // world
    lo = min(rows, per * rank) * PARAM_ALIGN
    hi = min(rows, per * (rank + 1)) * PARAM_ALIGN
    return lo, hi, per * PARAM_ALIGN


def _nbytes(t) -> int:
    return 0 if t is None else t.untyped_storage().nbytes()


def _release(t: torch.Tensor):
    t.untyped_storage().resize_(0)


def _materialize(t: torch.Tensor, nbytes: int):
    if t.untyped_storage().nbytes() != nbytes:
        t.untyped_storage().resize_(nbytes)


class DataParallel:
    name = "ddp"

    def __init__(self, opt: Optimizer, comm, model=None):
        self.opt, self.comm = opt, comm
        self.world, self.rank = comm.world, comm.rank

    def sync_params(self):
        self.comm.broadcast(self.opt.arena.val, 0)
        if self.opt.arena.shadow is not None:
            self.opt.arena.refresh_shadow()

    def begin_step(self):
        """Called before the forward / backward of a step (re-materialises what the previous step released)."""

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

    def full_values(self) -> torch.Tensor:
        """The whole fp32 value vector (arena order), for inspection / checkpoints."""
        a = self.opt.arena
        return a.val[: a.numel].clone()

    def state_bytes_per_rank(self):
        """Bytes of optimizer state actually allocated on this rank right now (values, gradients, moments)."""
        a = self.opt.arena
        return _nbytes(a.val) + _nbytes(a.grd) + _nbytes(a.m) + _nbytes(a.v)


class OverlappedDataParallel(DataParallel):
    """DDP whose gradient reduction overlaps the backward pass: the arena is cut into buckets of consecutive model
    units (walking from the end of the arena, the order in which the backward finishes gradients); every unit's
    ``vjp`` is wrapped, and as soon as the backward has passed the first unit of a bucket that bucket's slice of the
    gradient arena is reduced — asynchronously where the communicator can (NCCL: on its own stream, behind the
    kernels already enqueued, while the remaining backward runs).  ``reduce_grads`` only reduces what is left and
    waits.  Bit-identical to ``DataParallel``: the same elements are summed over the same ranks in the same order.
    Reference: GradReady / GradMarks + bucketed DDP (noeira/nn/distributed/grad_marks.mojo:75-379,
    noeira/nn/distributed/buckets.mojo, noeira/nn/distributed/data_parallel.mojo)."""
    name = "ddp_overlap"

    def __init__(self, opt: Optimizer, comm, model=None, bucket_bytes: int = 8 << 20):
        super().__init__(opt, comm, model)
        from .buckets import BucketedReducer, GradMarks, plan_buckets
        a = opt.arena
        units, ranges = self._units(a, model)
        gm = GradMarks()
        for i, (lo, hi) in enumerate(ranges):
            gm.add(f"unit{i}", lo, hi)
        self.buckets = plan_buckets(gm.marks, max(bucket_bytes // 4, 1))
        self._pending = []
        self.reducer = BucketedReducer(self.buckets, self._reduce_range)
        self.launched_during_backward = 0
        self._in_backward = False
        self.hooked = bool(units)
        for i, child in enumerate(units):
            self._hook(child, f"unit{i}")

    @staticmethod
    def _units(a, model):
        """The model's direct children that own parameters, with their arena ranges — when the arena order is the
        children's registration order (it is for every model built through ``add_child``); otherwise one unit."""
        kids = []
        if model is not None:
            kids = list(getattr(model, "mods", None) or getattr(model, "_children", {}).values())
            kids = [c for c in kids if list(c.params())]
        ents, out, i = a.entries, [], 0
        for child in kids:
            ids = {id(p) for p in child.params()}
            lo = ents[i][2] if i < len(ents) else a.numel
            n0 = i
            while i < len(ents) and id(ents[i][1]) in ids:
                i += 1
            if i == n0:
                return [], [(0, a.numel)]
            out.append((lo, ents[i][2] if i < len(ents) else a.numel))
        if not kids or i != len(ents):
            return [], [(0, a.numel)]
        return kids, out

    def _reduce_range(self, begin: int, end: int):
        view = self.opt.arena.grd[begin:end]
        if self._in_backward:
            self.launched_during_backward += 1
        if hasattr(self.comm, "all_reduce_async"):
            self._pending.append(self.comm.all_reduce_async(view))
        else:
            self.comm.all_reduce(view)

    def _hook(self, child, name):
        vjp = child.vjp

        def backward(*args, **kw):
            self._in_backward = True
            try:
                out = vjp(*args, **kw)
            finally:
                self._in_backward = False
            self._in_backward = True
            self.reducer.on_unit_done(name)      # this unit's gradients are complete: its bucket may go
            self._in_backward = False
            return out

        child.vjp = backward

    def reduce_grads(self):
        self.reducer.finish()
        for w in self._pending:
            w.wait()
        self._pending.clear()
        self.opt.arena.grd.mul_(1.0 / self.world)


class _ShardState:
    """Shard-size Adam state of one contiguous arena range ``[lo, lo + per·world)`` split over the ranks."""

    def __init__(self, val_full: torch.Tensor, flags_rows: torch.Tensor, per: int, rank: int, world: int, m_full=None, v_full=None):
        dev = val_full.device
        s = slice(rank * per, (rank + 1) * per)
        self.per, self.rank, self.world = per, rank, world
        self.m = torch.zeros(per, dtype=torch.float32, device=dev)
        self.v = torch.zeros(per, dtype=torch.float32, device=dev)
        if m_full is not None:
            k = min(per, max(0, m_full.numel() - rank * per))
            self.m[:k].copy_(m_full[rank * per: rank * per + k])
            self.v[:k].copy_(v_full[rank * per: rank * per + k])
        self.g = torch.zeros(per, dtype=torch.float32, device=dev)
        # per-element flags of the shard, expanded ONCE (bit 0 = weight decay, bit 1 = frozen); rows beyond the
        # arena are padding: frozen
        fl = torch.full((per * world // PARAM_ALIGN,), 2, dtype=torch.uint8, device=flags_rows.device)
        fl[: flags_rows.numel()] = flags_rows
        self.flags = fl.repeat_interleave(PARAM_ALIGN)[s].to(dev)
        live = (self.flags & 2) == 0
        self.masks = (bool(live.all()), live, ((self.flags & 1) != 0).to(torch.float32))

    def adam(self, val_shard: torch.Tensor, hyper: torch.Tensor):
        """AdamW on the shard with exactly the arithmetic of the arena optimizer (same helper, same scalars)."""
        lr, b1, b2, eps, wd, b1t, b2t, gs = (float(hyper[i]) for i in (H_LR, H_BETA1, H_BETA2, H_EPS, H_WD, H_B1T, H_B2T, H_GSCALE))
        g = self.g if gs == 1.0 else self.g * gs
        adamw_update_cpu(val_shard, g, self.m, self.v, None, lr, b1, b2, eps, wd, b1t, b2t, masks=self.masks)

    def nbytes(self):
        return _nbytes(self.m) + _nbytes(self.v) + _nbytes(self.g)


def _advance(hyper):
    hyper[H_T] += 1
    hyper[H_B1T] *= hyper[H_BETA1]
    hyper[H_B2T] *= hyper[H_BETA2]


class Zero1(DataParallel):
    name = "zero1"
    release_grads = False

    def __init__(self, opt, comm, model=None):
        super().__init__(opt, comm)
        a = opt.arena
        self.lo, self.hi, self.per = shard_range(a.numel, self.world, self.rank)
        self.padded = self.per * self.world
        a.repad(self.padded)                                   # collectives run in place on the arena
        self.shard = _ShardState(a.val, a.row_flags, self.per, self.rank, self.world, a.m, a.v)
        a.release_moments()                                    # the full-size m / v are gone: 2Ψ floats freed
        self._grd_bytes = _nbytes(a.grd)

    def _slice(self):
        return slice(self.rank * self.per, (self.rank + 1) * self.per)

    def begin_step(self):
        a = self.opt.arena
        if _nbytes(a.grd) != self._grd_bytes:
            _materialize(a.grd, self._grd_bytes)
            a.grd.zero_()

    def reduce_grads(self):
        a = self.opt.arena
        self.comm.reduce_scatter(self.shard.g, a.grd)
        self.shard.g.mul_(1.0 / self.world)
        if self.release_grads:
            _release(a.grd)                                    # ZeRO-2: only the shard survives the reduce-scatter

    def grad_norm(self):
        t = self.shard.g.double().pow(2).sum().reshape(1).float()
        self.comm.all_reduce(t)
        return float(t.sqrt())

    def clip_grads(self, max_norm):
        n = self.grad_norm()
        s = 0.0 if not math.isfinite(n) else (max_norm / (n + 1e-6) if n > max_norm > 0 else 1.0)
        self.shard.g.mul_(s)
        return n

    def step(self):
        a = self.opt.arena
        _advance(self.opt.hyper)
        mine = a.val[self._slice()]
        self.shard.adam(mine, self.opt.hyper)
        self.comm.all_gather(a.val, mine.clone())
        if _nbytes(a.grd):
            a.grd.zero_()
        a.bump_versions(shadow_fresh=False)
        if a.shadow is not None:
            a.refresh_shadow()

    def state_bytes_per_rank(self):
        a = self.opt.arena
        return _nbytes(a.val) + _nbytes(a.grd) + self.shard.nbytes()


class Zero2(Zero1):
    """ZeRO-1 whose full gradient arena does not outlive the reduce-scatter."""
    name = "zero2"
    release_grads = True


class Zero3(DataParallel):
    """Parameters, gradients and moments sharded per unit; values are materialised around each unit's forward and
    backward only.  ``model``: a module with ``mods`` (e.g. ``nn.Sequential``); its children are the units (their
    parameters are contiguous in the arena because the arena follows the module walk).  Without a model there is
    one unit, gathered by ``gather_params`` and released by ``release_params``."""
    name = "zero3"

    def __init__(self, opt, comm, model=None):
        super().__init__(opt, comm)
        a = opt.arena
        groups = self._unit_ranges(a, model)
        flags = a.row_flags
        self.units: List[dict] = []
        dev = a.val.device
        for lo, hi, ents in groups:
            _, _, per = shard_range(hi - lo, self.world, 0)
            full_v = torch.zeros(per * self.world, dtype=torch.float32, device=dev)
            full_g = torch.zeros(per * self.world, dtype=torch.float32, device=dev)
            full_v[: hi - lo].copy_(a.val[lo:hi])
            m_full = a.m[lo:hi] if a.m is not None else None
            v_full = a.v[lo:hi] if a.v is not None else None
            st = _ShardState(full_v, flags[lo // PARAM_ALIGN: hi // PARAM_ALIGN], per, self.rank, self.world, m_full, v_full)
            u = dict(lo=lo, hi=hi, per=per, full_v=full_v, full_g=full_g, state=st, nbytes=full_v.untyped_storage().nbytes(),
                     val_shard=full_v[self.rank * per:(self.rank + 1) * per].clone(), ents=ents, live_v=True, live_g=True)
            for _, p, o, n in ents:                              # parameters now view the unit's own buffers
                p._val = full_v[o - lo:o - lo + n].view(p.storage_shape)
                p._grd = full_g[o - lo:o - lo + n].view(p.storage_shape)
                p._shadow = None
            self.units.append(u)
        # the monolithic arena buffers are gone
        a.release_moments()
        for t in (a.val, a.grd):
            _release(t)
        if a.shadow is not None:
            _release(a.shadow)
            a.shadow = None
        self.gathered = True
        if model is not None and hasattr(model, "mods") and len(groups) == len(model.mods):
            for u, child in zip(self.units, model.mods):
                self._hook(child, u)
            self.hooked = True
            self.release_params()
        else:
            self.hooked = False

    @staticmethod
    def _unit_ranges(a, model):
        ents = a.entries
        if model is None or not hasattr(model, "mods"):
            return [(0, a.numel, list(ents))]
        out, i = [], 0
        for child in model.mods:
            ids = {id(p) for p in child.params()}
            mine = []
            while i < len(ents) and id(ents[i][1]) in ids:
                mine.append(ents[i])
                i += 1
            if mine:
                lo = mine[0][2]
                hi = ents[i][2] if i < len(ents) else a.numel
                out.append((lo, hi, mine))
        if i != len(ents) or len(out) != len([c for c in model.mods if list(c.params())]):
            return [(0, a.numel, list(ents))]                   # walk order does not match: fall back to one unit
        return out

    # ---- unit life cycle
    def _gather_unit(self, u):
        if not u["live_v"]:
            _materialize(u["full_v"], u["nbytes"])
            u["live_v"] = True
        self.comm.all_gather(u["full_v"], u["val_shard"])
        for _, p, _, _ in u["ents"]:
            p.version += 1

    def _release_unit(self, u):
        if u["live_v"]:
            _release(u["full_v"])
            u["live_v"] = False

    def _materialize_grads(self, u):
        if not u["live_g"]:
            _materialize(u["full_g"], u["nbytes"])
            u["full_g"].zero_()
            u["live_g"] = True

    def _reduce_scatter_unit(self, u):
        self.comm.reduce_scatter(u["state"].g, u["full_g"])
        u["state"].g.mul_(1.0 / self.world)
        _release(u["full_g"])
        u["live_g"] = False

    def _hook(self, child, u):
        fwd, vjp = child.forward, child.vjp

        def forward(*args, **kw):                               # PRE_FORWARD gather, POST_FORWARD release
            self._gather_unit(u)
            try:
                return fwd(*args, **kw)
            finally:
                self._release_unit(u)

        def backward(*args, **kw):                              # PRE_VJP gather, POST_VJP reduce-scatter + release
            self._gather_unit(u)
            self._materialize_grads(u)
            try:
                return vjp(*args, **kw)
            finally:
                self._reduce_scatter_unit(u)
                self._release_unit(u)

        child.forward, child.vjp = forward, backward

    # ---- strategy interface
    def sync_params(self):
        for u in self.units:
            was = u["live_v"]
            if not was:
                _materialize(u["full_v"], u["nbytes"])
                u["live_v"] = True
                self.comm.all_gather(u["full_v"], u["val_shard"])
            self.comm.broadcast(u["full_v"], 0)
            u["val_shard"].copy_(u["full_v"][self.rank * u["per"]:(self.rank + 1) * u["per"]])
            if not was:
                self._release_unit(u)

    def gather_params(self):
        for u in self.units:
            self._gather_unit(u)
        self.gathered = True

    def release_params(self):
        for u in self.units:
            self._release_unit(u)
        self.gathered = False

    def begin_step(self):
        if not self.hooked:
            self.gather_params()
            for u in self.units:
                self._materialize_grads(u)

    def reduce_grads(self):
        if not self.hooked:
            for u in self.units:
                self._reduce_scatter_unit(u)

    def grad_norm(self):
        t = sum(u["state"].g.double().pow(2).sum() for u in self.units).reshape(1).float()
        self.comm.all_reduce(t)
        return float(t.sqrt())

    def clip_grads(self, max_norm):
        n = self.grad_norm()
        s = 0.0 if not math.isfinite(n) else (max_norm / (n + 1e-6) if n > max_norm > 0 else 1.0)
        for u in self.units:
            u["state"].g.mul_(s)
        return n

    def step(self):
        _advance(self.opt.hyper)
        for u in self.units:
            u["state"].adam(u["val_shard"], self.opt.hyper)
        if not self.hooked:
            self.release_params()

    def full_values(self) -> torch.Tensor:
        a = self.opt.arena
        out = torch.zeros(a.numel, dtype=torch.float32, device=self.units[0]["val_shard"].device)
        for u in self.units:
            full = torch.zeros(u["per"] * self.world, dtype=torch.float32, device=out.device)
            self.comm.all_gather(full, u["val_shard"])
            out[u["lo"]:u["hi"]].copy_(full[: u["hi"] - u["lo"]])
        return out

    def state_bytes_per_rank(self):
        return sum(_nbytes(u["full_v"]) + _nbytes(u["full_g"]) + _nbytes(u["val_shard"]) + u["state"].nbytes() for u in self.units)


STRATEGIES = {"ddp": DataParallel, "ddp_overlap": OverlappedDataParallel, "zero1": Zero1, "zero2": Zero2, "zero3": Zero3}
