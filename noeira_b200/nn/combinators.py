"""Combinators: chain forward / vjp of children and compose parameter paths
(noeira/nn/combinators/: sequential.mojo:24, residual.mojo:40, parallel.mojo:143, repeat.mojo:30,
tokenwise.mojo:26, checkpointed.mojo:39).  Path segments follow the reference: child index for
Sequential / Repeat / Parallel, ``0`` for Residual / Tokenwise, ``1`` for the projection of
ProjectedResidual."""
from __future__ import annotations

from typing import Callable, Sequence

import torch

from .layers import SAVES_OUTPUT, Linear
from .module import Module


class Sequential(Module):
    def __init__(self, *mods: Module):
        super().__init__()
        self.mods = list(mods)
        for i, m in enumerate(self.mods):
            self.add_child(i, m)

    def forward(self, x):
        for m in self.mods:
            x = m.forward(x)
        return x

    def vjp(self, g, fuse_dact=None):
        """Backward chain.  When layer i is a fused Linear+activation whose derivative can be evaluated
        from its saved tensor, that derivative is folded into layer i+1's dgrad GEMM epilogue."""
        n = len(self.mods)
        pre_flag = False
        for i in range(n - 1, -1, -1):
            m = self.mods[i]
            prev = self.mods[i - 1] if i > 0 else None
            fuse = None
            if isinstance(m, Linear) and m.need_input_grad:
                if isinstance(prev, Linear) and prev.act is not None and m.on_cuda and prev._saved is not None \
                        and prev._saved.dtype == torch.bfloat16 and prev._saved.shape[-1] % 8 == 0:
                    fuse = (prev.act, prev._saved)
                elif i == 0 and fuse_dact is not None:
                    fuse = fuse_dact
            if isinstance(m, Linear):
                g = m.vjp(g, dy_is_pre=pre_flag, fuse_dact=fuse)
                pre_flag = fuse is not None and i > 0
            elif hasattr(m, "lin") and isinstance(getattr(m, "lin"), Linear):
                if isinstance(prev, Linear) and prev.act is not None and m.on_cuda and prev._saved is not None \
                        and prev._saved.dtype == torch.bfloat16 and prev._saved.shape[-1] % 8 == 0:
                    fuse = (prev.act, prev._saved)
                g = m.vjp(g, fuse_dact=fuse)
                pre_flag = fuse is not None
            else:
                g = m.vjp(g)
                pre_flag = False
            if g is None:
                break
        return g


class Residual(Module):
    """y = x + inner(x); child path segment ``0``."""

    def __init__(self, inner: Module):
        super().__init__()
        self.inner = self.add_child(0, inner)

    def forward(self, x):
        return x + self.inner.forward(x)

    def vjp(self, g):
        return g + self.inner.vjp(g)


class ProjectedResidual(Module):
    """y = proj(x) + inner(x); inner at ``0``, projection at ``1``."""

    def __init__(self, inner: Module, proj: Module):
        super().__init__()
        self.inner = self.add_child(0, inner)
        self.proj = self.add_child(1, proj)

    def forward(self, x):
        return self.proj.forward(x) + self.inner.forward(x)

    def vjp(self, g):
        return self.proj.vjp(g) + self.inner.vjp(g)


class Parallel(Module):
    """Same input into every branch, outputs concatenated on the last axis (heads of a stochastic actor)."""

    def __init__(self, *mods: Module):
        super().__init__()
        self.mods = list(mods)
        for i, m in enumerate(self.mods):
            self.add_child(i, m)

    def forward(self, x):
        outs = [m.forward(x) for m in self.mods]
        self._widths = [o.shape[-1] for o in outs]
        return torch.cat([o.float() if o.dtype != outs[0].dtype else o for o in outs], dim=-1)

    def vjp(self, g):
        gs = torch.split(g, self._widths, dim=-1)
        total = None
        for m, gi in zip(self.mods, gs):
            d = m.vjp(gi.contiguous())
            total = d if total is None else total + d
        return total


class Repeat(Module):
    """N copies of a block in sequence (``shared=True`` ties the weights)."""

    def __init__(self, n: int, factory: Callable[[int], Module], shared: bool = False):
        super().__init__()
        if shared:
            blk = factory(0)
            self.mods = [blk] * n
            self.add_child(0, blk)
        else:
            self.mods = [factory(i) for i in range(n)]
            for i, m in enumerate(self.mods):
                self.add_child(i, m)
        self.shared = shared
        if shared and n > 1:
            raise NotImplementedError("weight-shared Repeat needs per-iteration activation caches")

    def forward(self, x):
        for m in self.mods:
            x = m.forward(x)
        return x

    def vjp(self, g):
        for m in reversed(self.mods):
            g = m.vjp(g)
        return g


class RepeatConditional(Module):
    """Residual stream chained through N layers that all receive the same conditioning inputs; the
    conditioning gradient is accumulated over layers (noeira/nn/combinators/repeat_conditional.mojo:56)."""

    def __init__(self, n: int, factory: Callable[[int], Module]):
        super().__init__()
        self.mods = [factory(i) for i in range(n)]
        for i, m in enumerate(self.mods):
            self.add_child(i, m)

    def forward(self, x, *cond):
        for m in self.mods:
            x = m.forward(x, *cond)
        return x

    def vjp(self, g):
        gc_total = None
        for m in reversed(self.mods):
            out = m.vjp(g)
            g, gc = out[0], out[1:]
            if gc_total is None:
                gc_total = list(gc)
            else:
                gc_total = [a if b is None else (b if a is None else a + b) for a, b in zip(gc_total, gc)]
        return (g, *gc_total)


class Tokenwise(Module):
    """Apply ``inner`` to every token of ``[B, SEQ, D]`` by folding SEQ into the batch; path segment ``0``."""

    def __init__(self, inner: Module):
        super().__init__()
        self.inner = self.add_child(0, inner)

    def forward(self, x):
        self._shape = x.shape
        y = self.inner.forward(x.reshape(-1, x.shape[-1]))
        return y.reshape(*self._shape[:-1], y.shape[-1])

    def vjp(self, g):
        d = self.inner.vjp(g.reshape(-1, g.shape[-1]))
        return None if d is None else d.reshape(*self._shape[:-1], d.shape[-1])


class SkipConcat(Module):
    """y = [x | inner(x)]"""

    def __init__(self, inner: Module):
        super().__init__()
        self.inner = self.add_child(0, inner)

    def forward(self, x):
        self._w = x.shape[-1]
        return torch.cat([x, self.inner.forward(x).to(x.dtype)], dim=-1)

    def vjp(self, g):
        return g[..., : self._w] + self.inner.vjp(g[..., self._w:].contiguous())


class StopGradParams(Module):
    """Forward and input gradient pass through, parameter gradients of ``inner`` are discarded
    (critics inside an actor loss, noeira/nn/combinators/: StopGradParams :103)."""

    def __init__(self, inner: Module):
        super().__init__()
        self.inner = inner  # deliberately NOT a registered child: not walked, not optimized here

    def forward(self, *x):
        return self.inner.forward(*x)

    def vjp(self, g):
        ps = self.inner.params()
        frozen = [p.frozen for p in ps]
        for p in ps:
            p.frozen = True
        try:
            return self.inner.vjp(g)
        finally:
            for p, f in zip(ps, frozen):
                p.frozen = f


class Checkpointed(Module):
    """Activation checkpointing: drop the inner caches after forward, recompute before vjp."""

    def __init__(self, inner: Module):
        super().__init__()
        self.inner = self.add_child(0, inner)

    def forward(self, *x):
        self._in = x
        y = self.inner.forward(*x)
        self.inner.release_buffers()
        return y

    def vjp(self, g):
        self.inner.forward(*self._in)
        return self.inner.vjp(g)


class StochasticActor(Module):
    """trunk (Sequential) + heads = Parallel(Linear μ, Linear ln σ) → packed ``[μ | ln σ]``
    (noeira/deep_agents/primitives/stochastic_actor.mojo:34-110)."""

    def __init__(self, trunk: Module, hidden: int, act_dim: int):
        super().__init__()
        self.trunk = self.add_child("trunk", trunk)
        self.heads = self.add_child("heads", Parallel(Linear(hidden, act_dim, out_fp32=True),
                                                     Linear(hidden, act_dim, out_fp32=True)))
        self.act_dim = act_dim

    def forward(self, x):
        return self.heads.forward(self.trunk.forward(x))

    def vjp(self, g):
        return self.trunk.vjp(self.heads.vjp(g))
