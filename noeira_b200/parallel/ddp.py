"""Data parallelism over the gradient arena.

Because all gradients of an optimizer already live in one contiguous arena, DDP needs no per-module
hooks: a bucket is a byte range of ``arena.grd`` (noeira/nn/distributed/data_parallel.mojo:190-202).
``FusedGradSync.reduce_and_step(opt)`` replaces ``all_reduce → scale → clip → Adam → bf16 recast →
zero_grad`` by ONE kernel that reads every peer's gradient arena over NVLink and applies the update
(csrc/allreduce_fused.cu).  ``NcclGradSync`` is the library baseline and test oracle.
"""
from __future__ import annotations

import ctypes
from typing import Dict

import torch
import torch.distributed as dist

from .._native import check, cuda_lib, ptr, stream_ptr
from ..nn.optim import H_GSCALE
from ..ops.status import device_status
from .symm import SIGNAL_PAD_WORDS, SymmetricHeap

ONE_SHOT, TWO_SHOT, MULTIMEM, PUSH = 0, 1, 2, 3
PUSH_MAX_OUT_BYTES = 16 << 20      # push sends (N-1) x bytes per GPU: beyond this the two-shot form moves fewer bytes
PUSH_MAX_BLOCKS = 1024


def choose_algo(nbytes: int, world: int, have_multicast: bool = False) -> int:
    """Per-bucket choice among the barrier-based forms (the push form, one NVLink traversal and no barrier, is chosen
    by ``FusedGradSync`` for whole groups of small arenas).  One-shot moves (N-1)·bytes per GPU but has the fewest flag rounds; two-shot
    moves 2(N-1)/N·bytes; multimem ≈ 2·bytes/N.  Crossovers follow timings on 8 B200s: one-shot wins up to
    512 KB, two-shot (or multimem, when a multicast mapping exists) above."""
    if world <= 2 or nbytes <= (512 << 10):
        return ONE_SHOT
    if have_multicast and nbytes >= (4 << 20):
        return MULTIMEM
    return TWO_SHOT


class NcclGradSync:
    """Baseline: NCCL all-reduce on the gradient arena, then the local arena optimizer."""

    def __init__(self, world, rank):
        self.world, self.rank = world, rank

    def attach(self, *opts):
        for o in opts:
            o.grad_scale = 1.0 / self.world
            o.hyper[H_GSCALE] = 1.0 / self.world

    def reduce_and_step(self, opt):
        dist.all_reduce(opt.arena.grd)
        if opt.max_grad_norm > 0:
            opt.clip(base_scale=1.0 / self.world)
        opt.step(zero_grad=True)


class FusedGradSync:
    """One-shot / two-shot / multimem gradient reduction fused with the optimizer update."""

    def __init__(self, world: int, rank: int, local_rank: int, group=None, algo: int = None, spin_limit: int = 1 << 24):
        self.world, self.rank, self.local_rank, self.group = world, rank, local_rank, group
        self.algo = algo
        self.spin_limit = spin_limit
        self.state: Dict[int, dict] = {}
        self.lib = cuda_lib()
        self.sig_heap = None
        self.opts = []
        self.push = None

    def attach(self, *opts):
        """Move each optimizer's gradient arena into symmetric memory and build the peer tables."""
        total = 0
        for o in opts:
            total += 2 * (o.arena.numel * 4 + 512)
        total += 4 * SIGNAL_PAD_WORDS * len(opts) + 4096
        self.heap = SymmetricHeap(total, self.group)
        for o in opts:
            a = o.arena
            g = self.heap.tensor(a.numel, torch.float32)
            r = self.heap.tensor(a.numel, torch.float32)
            s = self.heap.tensor(SIGNAL_PAD_WORDS, torch.int32)
            g.local.copy_(a.grd)
            # re-point the arena and every parameter's gradient view
            a.grd = g.local
            for _, p, off, n in a.entries:
                p._grd = a.grd[off:off + n].view(p.storage_shape)
            o.grad_scale = 1.0 / self.world
            o.hyper[H_GSCALE] = 1.0 / self.world
            nbytes = a.numel * 4
            self.state[id(o)] = dict(grd=g, red=r, sig=s, grd_tab=g.ptr_table(), red_tab=r.ptr_table(),
                                     sig_tab=s.ptr_table(),
                                     partials=torch.zeros(256, device=a.grd.device),
                                     algo=self.algo if self.algo in (ONE_SHOT, TWO_SHOT, MULTIMEM)
                                     else choose_algo(nbytes, self.world))
        self.opts = list(opts)
        self._setup_push()
        torch.cuda.synchronize()
        if dist.is_initialized():
            dist.barrier(group=self.group)

    # ------------------------------------------------------------------ push form (small arenas, one launch for all)
    def _setup_push(self):
        """Inbox + flags for the latency-optimal push all-reduce over ALL attached optimizers in one launch; used
        when their arenas together are small enough that sending (N-1) copies beats the two-shot form."""
        self.push = None
        if self.algo not in (None, PUSH) or not (1 <= len(self.opts) <= 4):
            return
        nblk = [self.lib.nb_push_blocks(ctypes.c_longlong(o.arena.numel)) for o in self.opts]
        plane = sum(nblk) * 1024 * 4                   # floats per (parity, source) plane
        if sum(nblk) > PUSH_MAX_BLOCKS or (self.algo is None and plane * 4 * (self.world - 1) > PUSH_MAX_OUT_BYTES):
            return
        heap = SymmetricHeap(2 * self.world * plane * 4 + 2 * self.world * PUSH_MAX_BLOCKS * 4 + 8192, self.group)
        inbox = heap.tensor(2 * self.world * plane, torch.float32)
        flags = heap.tensor(2 * self.world * PUSH_MAX_BLOCKS, torch.int32)
        dev = inbox.local.device
        self.push = dict(heap=heap, inbox=inbox, flags=flags, inbox_tab=inbox.ptr_table(), flag_tab=flags.ptr_table(),
                         ctl=torch.zeros(4, dtype=torch.int32, device=dev), args={})

    def _push_args(self, opts, update: bool):
        key = (tuple(id(o) for o in opts), update)
        a = self.push["args"].get(key)
        if a is None:
            k = len(opts)
            P, F, L = ctypes.c_void_p * k, ctypes.c_void_p * k, ctypes.c_longlong * k
            arr = lambda ts: P(*[t.data_ptr() if t is not None else 0 for t in ts])
            ars = [o.arena for o in opts]
            a = dict(grd=arr([x.grd for x in ars]), n=L(*[x.numel for x in ars]), hyper=arr([o.hyper for o in opts]))
            if update:
                a.update(val=arr([x.val for x in ars]), m=arr([x.m for x in ars]), v=arr([x.v for x in ars]),
                         shadow=arr([x.shadow for x in ars]), flags=arr([x.row_flags for x in ars]), out=None)
            else:
                outs = [torch.zeros_like(x.grd) for x in ars]
                a.update(out=arr(outs), outs=outs, val=None, m=None, v=None, shadow=None, flags=None)
            self.push["args"][key] = a
        return a

    def _push_launch(self, opts, update: bool, zero_grad: bool):
        a, ps = self._push_args(opts, update), self.push
        check(self.lib.nb_allreduce_push(
            ctypes.c_int(self.world), ctypes.c_int(self.rank), ctypes.c_int(len(opts)), ps["inbox_tab"], ps["flag_tab"],
            ptr(ps["ctl"]), a["grd"], a["out"], a["val"], a["m"], a["v"], a["shadow"], a["flags"], a["hyper"], a["n"],
            ctypes.c_int(1 if update else 0), ctypes.c_int(int(zero_grad)), ctypes.c_uint(self.spin_limit),
            ptr(device_status(opts[0].arena.grd.device)), stream_ptr()), "allreduce_push")
        return a

    def reduce_and_step_many(self, opts):
        """Reduce the gradients of several optimizers across ranks and apply their updates.  When the push form is
        set up (small arenas, no gradient clipping) this is ONE kernel for all of them, Adam step counters included;
        otherwise one fused kernel per optimizer, in the given order on every rank."""
        opts = list(opts)
        if (self.push is not None and all(id(o) in self.state for o in opts) and set(map(id, opts)) == set(map(id, self.opts))
                and all(o.max_grad_norm <= 0 for o in opts)):
            self._push_launch(self.opts, update=True, zero_grad=True)
            for o in self.opts:
                o.arena.bump_versions(shadow_fresh=True)
            return
        for o in opts:
            self.reduce_and_step(o)

    def reduce_and_step(self, opt):
        if self.push is not None and len(self.opts) == 1 and opt is self.opts[0] and opt.max_grad_norm <= 0:
            return self.reduce_and_step_many([opt])
        st = self.state[id(opt)]
        a = opt.arena
        self._advance(opt)
        check(self.lib.nb_allreduce_fused(
            ctypes.c_int(st["algo"]), ctypes.c_int(self.world), ctypes.c_int(self.rank), st["grd_tab"], st["red_tab"],
            st["sig_tab"], ctypes.c_void_p(0), ctypes.c_void_p(0), ctypes.c_longlong(a.numel), ptr(a.val), ptr(a.m),
            ptr(a.v), ptr(a.shadow), ptr(a.row_flags), ptr(opt.hyper), ptr(st["partials"]), ptr(opt._norm),
            ctypes.c_float(opt.max_grad_norm), ctypes.c_int(1), ctypes.c_uint(self.spin_limit),
            ptr(device_status(a.grd.device)), stream_ptr()), "allreduce_fused")
        a.bump_versions(shadow_fresh=True)

    def _advance(self, opt):
        check(self.lib.nb_adam_advance(ptr(opt.hyper), stream_ptr()), "adam_advance")

    def all_reduce(self, opt, scale: float = None) -> torch.Tensor:
        """Plain fused all-reduce of the gradient arena (no update); returns the reduced arena view."""
        if self.push is not None and len(self.opts) == 1 and opt is self.opts[0] and self.algo in (None, PUSH):
            a = self._push_launch(self.opts, update=False, zero_grad=False)
            return a["outs"][0]
        st = self.state[id(opt)]
        a = opt.arena
        check(self.lib.nb_allreduce_fused(
            ctypes.c_int(st["algo"]), ctypes.c_int(self.world), ctypes.c_int(self.rank), st["grd_tab"], st["red_tab"],
            st["sig_tab"], ctypes.c_void_p(0), ctypes.c_void_p(0), ctypes.c_longlong(a.numel), None, None, None, None,
            None, ptr(opt.hyper) if scale is None else None, None, None, ctypes.c_float(0.0), ctypes.c_int(0),
            ctypes.c_uint(self.spin_limit), ptr(device_status(a.grd.device)), stream_ptr()), "allreduce_fused")
        return st["red"].local


class FusedZeroSync:
    """ZeRO-1 on GPUs as ONE kernel per step: reduce-scatter fused with the shard's AdamW, all-gather fused with the
    bf16 recast (``csrc/allreduce_fused.cu::ar_zero_kernel``).  Adam's moments exist only at shard size; gradients,
    values and the bf16 shadow live in symmetric memory so that peers read / write them directly.
    Reference: ``Zero1.reduce_scatter_grads`` + shard Adam + ``all_gather_rows`` noeira/nn/distributed/zero.mojo:284-402."""

    def __init__(self, world: int, rank: int, local_rank: int, group=None, spin_limit: int = 1 << 24):
        self.world, self.rank, self.local_rank, self.group, self.spin_limit = world, rank, local_rank, group, spin_limit
        self.lib = cuda_lib()
        self.lib.nb_zero_slice4.restype = ctypes.c_longlong
        self.state: Dict[int, dict] = {}

    def attach(self, *opts):
        for o in opts:
            a = o.arena
            if a.m is None:
                raise ValueError("the optimizer has no moments to shard")
            n = a.numel
            heap = SymmetricHeap(n * (4 + 4 + 2) + 4 * SIGNAL_PAD_WORDS + 4096, self.group)
            g, v = heap.tensor(n, torch.float32), heap.tensor(n, torch.float32)
            sh = heap.tensor(n, torch.bfloat16)
            sig = heap.tensor(SIGNAL_PAD_WORDS, torch.int32)
            g.local.copy_(a.grd)
            v.local.copy_(a.val)
            sh.local.copy_(a.val)
            a.grd, a.val, a.shadow = g.local, v.local, sh.local
            for _, p, off, k in a.entries:
                p._grd = a.grd[off:off + k].view(p.storage_shape)
                p._val = a.val[off:off + k].view(p.storage_shape)
                p._shadow = a.shadow[off:off + k].view(p.storage_shape)
                p.mark_shadow_fresh()
            per = 4 * int(self.lib.nb_zero_slice4(ctypes.c_longlong(n), ctypes.c_int(self.world)))
            lo = min(n, per * self.rank)
            hi = min(n, lo + per)
            m = torch.zeros(per, device=a.val.device)
            vv = torch.zeros(per, device=a.val.device)
            m[: hi - lo].copy_(a.m[lo:hi])
            vv[: hi - lo].copy_(a.v[lo:hi])
            a.release_moments()
            o.grad_scale = 1.0 / self.world
            o.hyper[H_GSCALE] = 1.0 / self.world
            self.state[id(o)] = dict(heap=heap, m=m, v=vv, per=per, grd_tab=g.ptr_table(), val_tab=v.ptr_table(),
                                     shadow_tab=sh.ptr_table(), sig_tab=sig.ptr_table())
        torch.cuda.synchronize()
        if dist.is_initialized():
            dist.barrier(group=self.group)

    def reduce_and_step(self, opt):
        if opt.max_grad_norm > 0:
            raise NotImplementedError("gradient clipping is not part of the fused ZeRO step; use parallel.strategy.Zero1")
        st, a = self.state[id(opt)], opt.arena
        check(self.lib.nb_adam_advance(ptr(opt.hyper), stream_ptr()), "adam_advance")
        check(self.lib.nb_zero_step_fused(
            ctypes.c_int(self.world), ctypes.c_int(self.rank), st["grd_tab"], st["val_tab"], st["shadow_tab"], st["sig_tab"],
            ctypes.c_longlong(a.numel), ptr(st["m"]), ptr(st["v"]), ptr(a.row_flags), ptr(opt.hyper), ctypes.c_int(1),
            ctypes.c_uint(self.spin_limit), ptr(device_status(a.grd.device)), stream_ptr()), "zero_step_fused")
        a.bump_versions(shadow_fresh=True)

    def state_bytes_per_rank(self, opt) -> int:
        st, a = self.state[id(opt)], opt.arena
        return a.numel * (4 + 4 + 2) + 2 * st["per"] * 4


class OverlapGradSync:
    """Gradient reduction overlapped with the backward pass: buckets of the gradient arena are all-reduced (NCCL, on
    the library's stream) as soon as the backward has finished their units, then the arena optimizer runs.  The
    trainer hands over its model with ``attach_model`` so that the units' ``vjp`` can be wrapped."""

    def __init__(self, world, rank, bucket_bytes: int = 8 << 20):
        self.world, self.rank, self.bucket_bytes = world, rank, bucket_bytes
        self.st = None
        self.opt = None

    def attach(self, *opts):
        assert len(opts) == 1, "one optimizer (one arena) per overlapped sync"
        self.opt = opts[0]

    def attach_model(self, model):
        from .fibers import DistComm
        from .strategy import OverlappedDataParallel
        self.st = OverlappedDataParallel(self.opt, DistComm(), model=model, bucket_bytes=self.bucket_bytes)

    def reduce_and_step(self, opt):
        assert self.st is not None, "attach_model(model) first"
        self.st.reduce_grads()
        if opt.max_grad_norm > 0:
            opt.clip()
        opt.step(zero_grad=True)


def make_grad_sync(kind: str, world: int, rank: int, local_rank: int):
    if kind == "nccl":
        return NcclGradSync(world, rank)
    if kind == "overlap":
        return OverlapGradSync(world, rank)
    if kind == "zero":
        return FusedZeroSync(world, rank, local_rank)
    return FusedGradSync(world, rank, local_rank)
