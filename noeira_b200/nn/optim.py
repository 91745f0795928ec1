"""Optimizers over a ParamArena: Adam / AdamW / SGD / LaProp and the scalar Adam used for the SAC
temperature.  Hyper-parameters, step count and beta powers live in a small device tensor
(``hyper``) so that a captured CUDA graph picks up schedule changes on replay
(noeira/nn/optimizer/adam.mojo:75-160: device resident β^t, lr from device memory).
Gradient clipping is the reference's three steps — Σg², finalize, scale — with the scale folded into
the update kernel instead of a separate pass (noeira/nn/optimizer/grad_clip.mojo:255-320); a
non-finite norm zeroes the step.
"""
from __future__ import annotations

import ctypes
import math
from typing import Iterable, Tuple

import torch

from .._native import check, cuda_lib, ptr, stream_ptr
from .arena import ParamArena
from .param import Param

H_LR, H_BETA1, H_BETA2, H_EPS, H_WD, H_T, H_B1T, H_B2T, H_GSCALE = range(9)
H_SIZE = 16


class Optimizer:
    def __init__(self, named_params: Iterable[Tuple[str, Param]], lr: float, device=None, tensor_factory=None,
                 with_moments=True):
        self.arena = ParamArena(list(named_params), device=device, with_moments=with_moments,
                                tensor_factory=tensor_factory)
        self.device = self.arena.device
        self.cuda = self.device.type == "cuda"
        self.hyper = torch.zeros(H_SIZE, dtype=torch.float32, device=self.device)
        self.max_grad_norm = 0.0
        self.grad_scale = 1.0
        self._sumsq = torch.zeros(1, device=self.device)
        self._norm = torch.zeros(1, device=self.device)
        self._partials = torch.zeros(2048, device=self.device)
        self._ticket = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._set(H_LR, lr)
        self._set(H_GSCALE, 1.0)

    def _set(self, idx, v):
        self.hyper[idx] = float(v)

    def set_lr(self, lr: float):
        self._set(H_LR, lr)

    def zero_grad(self):
        self.arena.zero_grad()

    def grad_norm(self) -> torch.Tensor:
        """Device scalar holding the (scaled) gradient norm measured at the last ``clip`` call."""
        return self._norm

    def clip(self, max_norm: float = None, base_scale: float = None):
        """Compute the global gradient norm on the device and fold the clip factor into hyper[GSCALE]."""
        mx = self.max_grad_norm if max_norm is None else max_norm
        bs = self.grad_scale if base_scale is None else base_scale
        a = self.arena
        if self.cuda:
            lib = cuda_lib()
            check(lib.nb_arena_sumsq(ptr(a.grd), ctypes.c_longlong(a.numel), ptr(self._partials), ptr(self._ticket),
                                     ptr(self._sumsq), stream_ptr()), "sumsq")
            check(lib.nb_clip_finalize(ptr(self._sumsq), ctypes.c_float(mx), ctypes.c_float(bs), ptr(self.hyper),
                                       ptr(self._norm), stream_ptr()), "clip_finalize")
        else:
            norm = a.grd.double().pow(2).sum().sqrt().item() * bs
            s = bs
            if not math.isfinite(norm):
                s = 0.0
            elif mx > 0 and norm > mx:
                s = bs * mx / (norm + 1e-6)
            self.hyper[H_GSCALE] = s
            self._norm[0] = norm

    def step(self, zero_grad: bool = False):
        raise NotImplementedError

    # checkpoint scalars (noeira/nn/optimizer/adam.mojo:353-380: t, β₁ᵗ, β₂ᵗ)
    def scalars(self):
        h = self.hyper.cpu()
        return {"t": float(h[H_T]), "b1t": float(h[H_B1T]), "b2t": float(h[H_B2T])}

    def load_scalars(self, d):
        self._set(H_T, d.get("t", 0.0))
        self._set(H_B1T, d.get("b1t", 1.0))
        self._set(H_B2T, d.get("b2t", 1.0))


def adamw_update_cpu(val, g, m, v, flags, lr, b1, b2, eps, wd, b1t, b2t, masks=None):
    """In-place AdamW on (views of) fp32 tensors; ``flags`` per element: bit 0 = weight decay, bit 1 = frozen.
    One arithmetic for every caller (arena optimizer, ZeRO shards): identical inputs give identical bits.
    ``masks`` = cached ``(all_live, live, decay)`` for the same flags."""
    if masks is None:
        live = (flags & 2) == 0
        masks = (bool(live.all()), live, ((flags & 1) != 0).to(val.dtype))
    all_live, live, decay = masks
    if not all_live:
        g = g * live.to(g.dtype)
        m_old, v_old, val_old = m.clone(), v.clone(), val.clone()
    m.mul_(b1).add_(g, alpha=1 - b1)
    v.mul_(b2).addcmul_(g, g, value=1 - b2)
    denom = (v / (1 - b2t)).sqrt_().add_(eps)
    if wd != 0.0:
        val.addcmul_(val, decay, value=-lr * wd)
    val.addcdiv_(m, denom, value=-lr / (1 - b1t))
    if not all_live:
        frozen = ~live
        m[frozen], v[frozen], val[frozen] = m_old[frozen], v_old[frozen], val_old[frozen]
    return masks


class AdamW(Optimizer):
    def __init__(self, named_params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, **kw):
        super().__init__(named_params, lr, **kw)
        self._set(H_BETA1, betas[0])
        self._set(H_BETA2, betas[1])
        self._set(H_EPS, eps)
        self._set(H_WD, weight_decay)
        self._set(H_T, 0.0)
        self._set(H_B1T, 1.0)
        self._set(H_B2T, 1.0)

    def step(self, zero_grad: bool = False):
        a = self.arena
        if self.cuda:
            lib = cuda_lib()
            check(lib.nb_adam_advance(ptr(self.hyper), stream_ptr()), "adam_advance")
            check(lib.nb_arena_adamw(ptr(a.val), ptr(a.grd), ptr(a.m), ptr(a.v), ptr(a.shadow), ptr(a.row_flags),
                                     ctypes.c_longlong(a.numel), ptr(self.hyper), ctypes.c_int(int(zero_grad)),
                                     stream_ptr()), "arena_adamw")
            a.bump_versions(shadow_fresh=True)
            return
        h = self.hyper
        h[H_T] += 1
        h[H_B1T] *= h[H_BETA1]
        h[H_B2T] *= h[H_BETA2]
        lr, b1, b2, eps, wd, b1t, b2t, gs = (float(h[i]) for i in (H_LR, H_BETA1, H_BETA2, H_EPS, H_WD, H_B1T, H_B2T, H_GSCALE))
        key = a.row_flags._version
        if getattr(self, "_cpu_masks_key", None) != key:
            flags = a.row_flags.repeat_interleave(32)[: a.numel]
            self._cpu_live = (flags & 2) == 0
            self._cpu_all_live = bool(self._cpu_live.all())
            self._cpu_decay = ((flags & 1) != 0).to(a.val.dtype)
            self._cpu_masks_key = key
        g = a.grd if gs == 1.0 else a.grd * gs
        adamw_update_cpu(a.val, g, a.m, a.v, None, lr, b1, b2, eps, wd, b1t, b2t,
                         masks=(self._cpu_all_live, self._cpu_live, self._cpu_decay))
        if zero_grad:
            a.grd.zero_()
        a.bump_versions(shadow_fresh=False)


_MULTI = {}


def step_many(opts, zero_grad: bool = True):
    """One Adam(W) step of several optimizers.  On CUDA (up to four AdamW-family optimizers without gradient clipping)
    this is ONE kernel that also advances their step counters; otherwise each optimizer steps on its own."""
    opts = list(opts)
    if (len(opts) < 2 or len(opts) > 4 or not all(type(o) in (AdamW, Adam) and o.cuda and o.max_grad_norm <= 0 for o in opts)):
        for o in opts:
            if o.max_grad_norm > 0:
                o.clip()
            o.step(zero_grad=zero_grad)
        return
    key = tuple(id(o) for o in opts)
    a = _MULTI.get(key)
    if a is None:
        k = len(opts)
        P, L = ctypes.c_void_p * k, ctypes.c_longlong * k
        arr = lambda ts: P(*[t.data_ptr() if t is not None else 0 for t in ts])
        ars = [o.arena for o in opts]
        a = dict(val=arr([x.val for x in ars]), m=arr([x.m for x in ars]), v=arr([x.v for x in ars]),
                 shadow=arr([x.shadow for x in ars]), flags=arr([x.row_flags for x in ars]), hyper=arr([o.hyper for o in opts]),
                 n=L(*[x.numel for x in ars]), ticket=torch.zeros(1, dtype=torch.int32, device=opts[0].device), ars=ars)
        _MULTI[key] = a
    # gradient arenas may have been re-pointed (e.g. into symmetric memory): read their addresses at call time
    grd = (ctypes.c_void_p * len(opts))(*[x.grd.data_ptr() for x in a["ars"]])
    check(cuda_lib().nb_arena_adamw_multi(ctypes.c_int(len(opts)), a["val"], grd, a["m"], a["v"], a["shadow"], a["flags"], a["hyper"],
                                          a["n"], ctypes.c_int(int(zero_grad)), ptr(a["ticket"]), stream_ptr()), "arena_adamw_multi")
    for x in a["ars"]:
        x.bump_versions(shadow_fresh=True)


class Adam(AdamW):
    def __init__(self, named_params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, **kw):
        super().__init__(named_params, lr=lr, betas=betas, eps=eps, weight_decay=0.0, **kw)


class SGD(Optimizer):
    def __init__(self, named_params, lr=1e-2, momentum=0.0, nesterov=False, weight_decay=0.0, **kw):
        super().__init__(named_params, lr, with_moments=momentum > 0, **kw)
        self.momentum, self.nesterov = momentum, nesterov
        self._set(H_WD, weight_decay)

    def step(self, zero_grad: bool = False):
        a = self.arena
        if self.cuda:
            check(cuda_lib().nb_arena_sgd(ptr(a.val), ptr(a.grd), ptr(a.m), ptr(a.shadow), ptr(a.row_flags),
                                          ctypes.c_longlong(a.numel), ptr(self.hyper), ctypes.c_float(self.momentum),
                                          ctypes.c_int(int(self.nesterov)), stream_ptr()), "arena_sgd")
            a.bump_versions(shadow_fresh=True)
        else:
            h = self.hyper
            flags = a.row_flags.repeat_interleave(32)[: a.numel]
            g = a.grd * float(h[H_GSCALE]) + torch.where((flags & 1) != 0, float(h[H_WD]) * a.val, torch.zeros_like(a.val))
            if a.m is not None:
                a.m.mul_(self.momentum).add_(g)
                g = g + self.momentum * a.m if self.nesterov else a.m
            a.val.sub_(torch.where((flags & 2) == 0, float(h[H_LR]) * g, torch.zeros_like(g)))
            a.bump_versions(shadow_fresh=False)
        if zero_grad:
            a.grd.zero_()


class LaProp(AdamW):
    """Dreamer-family optimizer: gradient normalised by sqrt(v) before the momentum
    (noeira/nn/optimizer/dreamer_opt.mojo:179)."""

    def step(self, zero_grad: bool = False):
        a = self.arena
        if self.cuda:
            lib = cuda_lib()
            check(lib.nb_adam_advance(ptr(self.hyper), stream_ptr()), "adam_advance")
            check(lib.nb_arena_laprop(ptr(a.val), ptr(a.grd), ptr(a.m), ptr(a.v), ptr(a.shadow), ptr(a.row_flags),
                                      ctypes.c_longlong(a.numel), ptr(self.hyper), stream_ptr()), "arena_laprop")
            a.bump_versions(shadow_fresh=True)
        else:
            h = self.hyper
            h[H_T] += 1
            h[H_B1T] *= h[H_BETA1]
            h[H_B2T] *= h[H_BETA2]
            lr, b1, b2, eps, wd, b1t, b2t, gs = (float(h[i]) for i in (H_LR, H_BETA1, H_BETA2, H_EPS, H_WD, H_B1T, H_B2T, H_GSCALE))
            flags = a.row_flags.repeat_interleave(32)[: a.numel]
            g = a.grd * gs
            a.v.mul_(b2).add_((1 - b2) * g * g)
            a.m.mul_(b1).add_((1 - b1) * g / ((a.v / (1 - b2t)).sqrt() + eps))
            upd = a.m / (1 - b1t) + torch.where((flags & 1) != 0, wd * a.val, torch.zeros_like(a.val))
            a.val.sub_(lr * upd)
            a.bump_versions(shadow_fresh=False)
        if zero_grad:
            a.grd.zero_()


class ScalarAdam:
    """Adam on one device-resident scalar (SAC's ln α): state = [ln α, m, v, β₁ᵗ, β₂ᵗ, α]
    (noeira/nn/optimizer/scalar_adam.mojo:73)."""

    def __init__(self, init_value: float, lr: float, device="cpu", betas=(0.9, 0.999), eps=1e-8):
        self.state = torch.tensor([math.log(init_value), 0.0, 0.0, 1.0, 1.0, init_value], dtype=torch.float32, device=device)
        self.lr, self.betas, self.eps = lr, betas, eps

    @property
    def alpha(self) -> torch.Tensor:
        return self.state[5]

    def step_alpha(self, mean_logp: torch.Tensor, target_entropy: float):
        if self.state.is_cuda:
            check(cuda_lib().nb_scalar_adam_alpha(ptr(self.state), ptr(mean_logp), ctypes.c_float(target_entropy),
                                                  ctypes.c_float(self.lr), ctypes.c_float(self.betas[0]),
                                                  ctypes.c_float(self.betas[1]), ctypes.c_float(self.eps), stream_ptr()),
                  "scalar_adam")
            return
        s = self.state
        g = -(float(mean_logp) + target_entropy)
        b1, b2 = self.betas
        s[3] *= b1
        s[4] *= b2
        s[1] = b1 * s[1] + (1 - b1) * g
        s[2] = b2 * s[2] + (1 - b2) * g * g
        s[0] -= self.lr * (s[1] / (1 - s[3])) / (math.sqrt(float(s[2] / (1 - s[4]))) + self.eps)
        s[5] = math.exp(float(s[0]))


def polyak(target_arena: ParamArena, online_arena: ParamArena, tau: float):
    """target ← target + τ (online − target) over the whole arena in one kernel
    (noeira/nn/optimizer/param_arena.mojo:250-288)."""
    if target_arena.val.is_cuda:
        check(cuda_lib().nb_polyak(ptr(target_arena.val), ptr(online_arena.val), ctypes.c_longlong(target_arena.numel),
                                   ctypes.c_float(tau), stream_ptr()), "polyak")
        if target_arena.shadow is not None:
            target_arena.refresh_shadow()
    else:
        target_arena.val.lerp_(online_arena.val, tau)
    target_arena.bump_versions(shadow_fresh=target_arena.shadow is not None)
