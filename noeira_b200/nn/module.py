"""Module base class: explicit forward / vjp pairs, no autograd tape.

Every leaf caches what its backward needs in ``forward`` and implements ``vjp(grad_out)`` that
(a) accumulates parameter gradients into ``Param.grad`` and (b) returns the gradient(s) of its
input(s).  Combinators chain children.  This mirrors the reference's ``Module`` trait
(noeira/nn/core/module.mojo:25-169: forward, vjp, for_each_param, zero_grad, for_each_state,
polyak_from, release_buffers, set_attr) with runtime shapes instead of compile-time ones.

Two execution targets, chosen by where the parameters live:
  * ``cuda`` — bf16 activation flow through the hand-written sm_100a kernels (``noeira_b200.ops``);
    a missing kernel library is an error, never a silent fallback;
  * ``cpu``  — fp32 PyTorch ops; this is the numerics oracle the GPU path is tested against.

Parameter naming: children are registered under a path segment (index for Sequential / Repeat /
Parallel, ``0`` for Residual / Tokenwise, node name for ComputeGraph) and ``named_params`` yields
dotted paths, e.g. ``actor.trunk.0.weight`` (noeira/nn/core/named_params.mojo:76).
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Callable, Iterator, Tuple

import torch

from .init import Initializer, Kaiming
from .param import Param, State

import threading

_TLS = threading.local()


def _gen() -> torch.Generator:
    """Per-thread initialisation stream (rank threads of the simulator must not interleave their draws)."""
    g = getattr(_TLS, "gen", None)
    if g is None:
        g = torch.Generator().manual_seed(0)
        _TLS.gen = g
    return g


def manual_seed(seed: int):
    """Seed the (CPU-side, deterministic) parameter initialisation stream of the calling thread."""
    _gen().manual_seed(int(seed))


class Module:
    ARITY = 1

    def __init__(self):
        self._params: "OrderedDict[str, Param]" = OrderedDict()
        self._states: "OrderedDict[str, State]" = OrderedDict()
        self._children: "OrderedDict[str, Module]" = OrderedDict()
        self.training = True
        self.attrs = {}
        self.device = torch.device("cpu")

    # ------------------------------------------------------------------ registration
    def add_param(self, name: str, shape, decay: bool = True, init: Initializer = None, fan_in: int = 1,
                  fan_out: int = 1, pad_rows: bool = True) -> Param:
        p = Param(name, shape, decay=decay, pad_rows=pad_rows)
        p.set_((init or Kaiming())(tuple(shape), fan_in, fan_out, _gen()))
        self._params[name] = p
        return p

    def add_state(self, name: str, shape, fill: float = 0.0) -> State:
        s = State(name, shape, fill=fill)
        self._states[name] = s
        return s

    def add_child(self, key, module: "Module") -> "Module":
        self._children[str(key)] = module
        return module

    # ------------------------------------------------------------------ traversal
    def named_params(self, prefix: str = "") -> Iterator[Tuple[str, Param]]:
        for n, p in self._params.items():
            yield prefix + n, p
        for k, c in self._children.items():
            yield from c.named_params(prefix + k + ".")

    def named_states(self, prefix: str = "") -> Iterator[Tuple[str, State]]:
        for n, s in self._states.items():
            yield prefix + n, s
        for k, c in self._children.items():
            yield from c.named_states(prefix + k + ".")

    def params(self):
        return [p for _, p in self.named_params()]

    def for_each_param(self, fn: Callable[[str, Param], None], prefix: str = ""):
        for n, p in self.named_params(prefix):
            fn(n, p)

    def for_each_state(self, fn: Callable[[str, State], None], prefix: str = ""):
        for n, s in self.named_states(prefix):
            fn(n, s)

    def modules(self):
        yield self
        for c in self._children.values():
            yield from c.modules()

    def num_params(self) -> int:
        return sum(p.numel for p in self.params())

    # ------------------------------------------------------------------ state management
    def to(self, device) -> "Module":
        device = torch.device(device)
        for m in self.modules():
            m.device = device
            for p in m._params.values():
                p.to(device)
            for s in m._states.values():
                s.to(device)
            m._moved(device)
        return self

    def _moved(self, device):
        pass

    def cuda(self):
        return self.to("cuda")

    @property
    def on_cuda(self) -> bool:
        return self.device.type == "cuda"

    def zero_grad(self):
        for p in self.params():
            p.zero_grad()

    def train(self, mode: bool = True):
        self.set_attr("training", mode)
        return self

    def eval(self):
        return self.train(False)

    def set_attr(self, name: str, value):
        """Runtime attribute propagated through every combinator
        (noeira/nn/core/module.mojo:135-152: training, capture_recast, rng_stream, multiplier, ...)."""
        for m in self.modules():
            if name == "training":
                m.training = bool(value)
            m.attrs[name] = value
            m._attr_changed(name, value)

    def _attr_changed(self, name, value):
        pass

    def polyak_from(self, other: "Module", tau: float):
        with torch.no_grad():
            for (_, p), (_, q) in zip(self.named_params(), other.named_params()):
                p.storage.lerp_(q.storage, tau)
                p.version += 1

    def copy_from(self, other: "Module"):
        with torch.no_grad():
            for (_, p), (_, q) in zip(self.named_params(), other.named_params()):
                p.storage.copy_(q.storage)
                p.version += 1
            for (_, s), (_, r) in zip(self.named_states(), other.named_states()):
                s.data.copy_(r.data)

    def release_buffers(self):
        """Drop cached activations (activation checkpointing, noeira/nn/combinators/checkpointed.mojo:39)."""
        for m in self.modules():
            m._release()

    def _release(self):
        pass

    # ------------------------------------------------------------------ compute
    def forward(self, *xs):
        raise NotImplementedError

    def vjp(self, *gs):
        raise NotImplementedError

    def __call__(self, *xs):
        return self.forward(*xs)

    def act_dtype(self):
        return torch.bfloat16 if self.on_cuda else torch.float32

    def display_label(self) -> str:
        return type(self).__name__

    def __repr__(self):
        lines = [self.display_label()]
        for k, c in self._children.items():
            sub = repr(c).split("\n")
            lines.append(f"  ({k}): " + sub[0])
            lines.extend("  " + s for s in sub[1:])
        return "\n".join(lines)


class AutogradBridge(torch.autograd.Function):
    """Lets a Module take part in a torch.autograd graph: forward → Module.forward,
    backward → Module.vjp (parameter gradients land in Param.grad, not in .grad of torch tensors)."""

    @staticmethod
    def forward(ctx, module, *xs):
        ctx.module = module
        out = module.forward(*xs)
        return out

    @staticmethod
    def backward(ctx, *gs):
        g = ctx.module.vjp(*gs)
        if not isinstance(g, (tuple, list)):
            g = (g,)
        return (None,) + tuple(g)


def as_autograd(module: Module, *xs):
    return AutogradBridge.apply(module, *xs)


class RecomputeBridge(torch.autograd.Function):
    """Re-entrant form of ``AutogradBridge`` for modules that are applied SEVERAL times inside one autograd graph (an
    unrolled latent model, a shared head): a module caches one set of activations, so each application keeps only its
    inputs and runs the module's forward again right before its ``vjp`` (activation checkpointing per application).
    Parameter gradients of all applications add up in ``Param.grad``."""

    @staticmethod
    def forward(ctx, module, anchor, *xs):
        ctx.module = module
        ctx.xs = tuple(x.detach() if torch.is_tensor(x) else x for x in xs)
        return module.forward(*ctx.xs)

    @staticmethod
    def backward(ctx, *gs):
        with torch.enable_grad():                 # layers skip saving activations when no backward can follow
            ctx.module.forward(*ctx.xs)
        with torch.no_grad():
            g = ctx.module.vjp(*gs)
        if not isinstance(g, (tuple, list)):
            g = (g,)
        g = tuple(g) + (None,) * (len(ctx.xs) - len(g))
        return (None, None) + tuple(gi if torch.is_tensor(x) and x.is_floating_point() else None for gi, x in zip(g, ctx.xs))


_ANCHOR = {}


def apply(module: Module, *xs):
    """``module(*xs)`` as a differentiable torch operation that may be repeated within one graph (see ``RecomputeBridge``).
    The parameters are not torch leaves, so an application on inputs that carry no gradient (an encoder on observations)
    would be cut out of the graph; a constant anchor that requires grad keeps it in."""
    dev = next((x.device for x in xs if torch.is_tensor(x)), torch.device("cpu"))
    a = _ANCHOR.get(dev)
    if a is None:
        a = _ANCHOR[dev] = torch.zeros((), device=dev, requires_grad=True)
    return RecomputeBridge.apply(module, a, *xs)
