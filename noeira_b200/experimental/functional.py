"""An eager mode for ``nn``: shapes are run-time values, the network is whatever code ran, and a tape records the operations
to differentiate them in reverse.

``nn`` modules carry their own backward (``forward`` / ``vjp``) and fix their wiring when they are built.  This is the other
mode: ``Tape`` owns named parameters (``nn.Param`` objects, so the arena optimizers and the checkpoint writers of ``nn`` take
a tape where they take a module), ``FTensor`` is a handle on a tape node with the usual operators, ``F`` holds the fused
and the composite operations, and ``Tape.module`` runs an ``nn`` module as one node through its own ``forward`` / ``vjp``.
The reverse pass walks the nodes from the last to the first and dispatches on the node's operation tag; ``reset`` drops
the nodes of a step and keeps the parameters; ``no_grad`` records nothing.

On CUDA the fused ``F.linear`` node and ``@`` of aligned matrices run on the tcgen05 GEMM in TF32 mode (fp32 operands,
fp32 accumulation, bias and activation in the epilogue), exactly the launches of ``nn.Linear`` with ``precision="tf32"``;
everything else is tensor arithmetic on the node values.

Reference: noeira/experimental/functional/ (tape.mojo, ftensor.mojo, F.mojo, nd.mojo, extra.mojo, module_op.mojo).
"""
from __future__ import annotations

import contextlib
import math
import zlib
from typing import Dict, Iterator, List, Optional, Sequence, Tuple

import torch

from ..nn.param import Param

_ACT = {
    "relu": (torch.relu, lambda x, y: (y > 0).to(y.dtype)),
    "tanh": (torch.tanh, lambda x, y: 1 - y * y),
    "sigmoid": (torch.sigmoid, lambda x, y: y * (1 - y)),
    "silu": (torch.nn.functional.silu, lambda x, y: torch.sigmoid(x) * (1 + x * (1 - torch.sigmoid(x)))),
    "gelu": (lambda x: torch.nn.functional.gelu(x, approximate="tanh"), None),
}


def _gelu_grad(x):
    c = math.sqrt(2.0 / math.pi)
    u = c * (x + 0.044715 * x ** 3)
    t = torch.tanh(u)
    return 0.5 * (1 + t) + 0.5 * x * (1 - t * t) * c * (1 + 3 * 0.044715 * x * x)


def _unbroadcast(g: torch.Tensor, shape: Sequence[int]) -> torch.Tensor:
    """Sum a gradient over the axes numpy broadcasting added or stretched."""
    while g.dim() > len(shape):
        g = g.sum(0)
    for i, n in enumerate(shape):
        if n == 1 and g.shape[i] != 1:
            g = g.sum(i, keepdim=True)
    return g


def _use_gemm(*mats) -> bool:
    return all(m.is_cuda and m.dtype == torch.float32 and m.dim() == 2 and m.is_contiguous() and m.shape[0] % 8 == 0 and
               m.shape[1] % 8 == 0 for m in mats)


def _mm(a, b):
    """a [M, K] @ b [K, N]"""
    if _use_gemm(a, b):
        from .. import ops
        return ops.gemm(a, b, b_mn=True)
    return a @ b


def _mm_tn(a, b):
    """aᵀ @ b with a [K, M], b [K, N]"""
    if _use_gemm(a, b):
        from .. import ops
        return ops.gemm(a, b, a_mn=True, b_mn=True)
    return a.transpose(-1, -2) @ b


def _mm_nt(a, b):
    """a @ bᵀ with a [M, K], b [N, K]"""
    if _use_gemm(a, b):
        from .. import ops
        return ops.gemm(a, b)
    return a @ b.transpose(-1, -2)


class _Node:
    __slots__ = ("op", "inputs", "value", "grad", "saved", "param", "needs_grad")

    def __init__(self, op, inputs, value, saved=None, param=None, needs_grad=True):
        self.op, self.inputs, self.value, self.saved, self.param = op, inputs, value, saved, param
        self.grad: Optional[torch.Tensor] = None
        self.needs_grad = needs_grad

    @property
    def v(self) -> torch.Tensor:
        """Parameters read their live storage: an optimizer step is seen by the next forward."""
        return self.param.data if self.param is not None else self.value


class FTensor:
    """A handle on a tape node."""

    def __init__(self, tape: "Tape", node: _Node):
        self.tape, self.node = tape, node

    # ---- data
    @property
    def value(self) -> torch.Tensor:
        return self.node.v

    @property
    def grad(self) -> Optional[torch.Tensor]:
        return self.node.param.grad if self.node.param is not None else self.node.grad

    @property
    def shape(self):
        return tuple(self.value.shape)

    def item(self) -> float:
        return float(self.value)

    def backward(self, seed: torch.Tensor = None):
        self.tape.backward(self, seed)

    # ---- operators
    def _lift(self, o) -> "FTensor":
        return o if isinstance(o, FTensor) else self.tape.constant(o)

    def __add__(self, o):
        o = self._lift(o)
        return self.tape._record("add", (self, o), self.value + o.value)

    __radd__ = __add__

    def __sub__(self, o):
        o = self._lift(o)
        return self.tape._record("sub", (self, o), self.value - o.value)

    def __rsub__(self, o):
        return self._lift(o) - self

    def __mul__(self, o):
        o = self._lift(o)
        return self.tape._record("mul", (self, o), self.value * o.value)

    __rmul__ = __mul__

    def __truediv__(self, o):
        o = self._lift(o)
        return self.tape._record("div", (self, o), self.value / o.value)

    def __rtruediv__(self, o):
        return self._lift(o) / self

    def __neg__(self):
        return self.tape._record("neg", (self,), -self.value)

    def __pow__(self, p: float):
        return self.tape._record("pow", (self,), self.value ** p, saved=float(p))

    def __matmul__(self, o):
        o = self._lift(o)
        a, b = self.value, o.value
        return self.tape._record("matmul", (self, o), _mm(a, b) if a.dim() == 2 and b.dim() == 2 else a @ b)

    def T(self):
        return self.transpose(-1, -2)

    def transpose(self, a: int, b: int):
        return self.tape._record("transpose", (self,), self.value.transpose(a, b), saved=(a, b))

    def permute(self, *dims):
        return self.tape._record("permute", (self,), self.value.permute(*dims), saved=tuple(dims))

    def reshape(self, *shape):
        return self.tape._record("reshape", (self,), self.value.reshape(*shape), saved=self.shape)

    def narrow(self, dim: int, start: int, length: int):
        return self.tape._record("narrow", (self,), self.value.narrow(dim, start, length), saved=(dim, start, length, self.shape))

    def sum(self, axis=None, keepdim=False):
        v = self.value.sum() if axis is None else self.value.sum(axis, keepdim=keepdim)
        return self.tape._record("sum", (self,), v, saved=(axis, keepdim, self.shape))

    def mean(self, axis=None, keepdim=False):
        v = self.value.mean() if axis is None else self.value.mean(axis, keepdim=keepdim)
        return self.tape._record("mean", (self,), v, saved=(axis, keepdim, self.shape))

    def sum_rows(self):
        """[rows, cols] → [1, cols] (the bias-gradient reduction)."""
        return self.sum(0, keepdim=True)

    def max(self, axis: int, keepdim=False):
        v, idx = self.value.max(axis, keepdim=True)
        return self.tape._record("max", (self,), v if keepdim else v.squeeze(axis), saved=(axis, keepdim, idx, self.shape))

    def _unary(self, op, v, saved=None):
        return self.tape._record(op, (self,), v, saved=saved)

    def exp(self):
        return self._unary("exp", torch.exp(self.value))

    def log(self):
        return self._unary("log", torch.log(self.value))

    def sqrt(self):
        return self._unary("sqrt", torch.sqrt(self.value))

    def clamp(self, lo=None, hi=None):
        return self._unary("clamp", self.value.clamp(lo, hi), saved=(lo, hi))

    def act(self, name: str):
        return self._unary("act", _ACT[name][0](self.value), saved=name)

    def relu(self):
        return self.act("relu")

    def tanh(self):
        return self.act("tanh")

    def sigmoid(self):
        return self.act("sigmoid")

    def gelu(self):
        return self.act("gelu")

    def silu(self):
        return self.act("silu")

    def softmax(self, axis: int = -1):
        return self._unary("softmax", torch.softmax(self.value, axis), saved=axis)

    def log_softmax(self, axis: int = -1):
        return self._unary("log_softmax", torch.log_softmax(self.value, axis), saved=axis)


class FModule:
    """An ``nn`` module owned by a tape and called as one node: its ``forward`` runs in the forward pass, its ``vjp`` in the
    reverse pass (which also leaves the module's parameter gradients in their ``Param.grad``).  One call per step: a module
    keeps the activations of its latest forward."""

    def __init__(self, tape: "Tape", module, name: str):
        self.tape, self.module, self.name = tape, module, name

    def __call__(self, *xs: FTensor) -> FTensor:
        # on CUDA the activations of ``nn`` modules are bf16 rows (their kernels read nothing else); the tape's are fp32
        cuda = self.tape.device.type == "cuda"
        y = self.module.forward(*[(x.value.to(torch.bfloat16) if cuda and x.value.is_floating_point() else x.value) for x in xs])
        return self.tape._record("module", tuple(xs), y.float() if y.dtype != torch.float32 else y, saved=self.module, force=True)


class Tape:
    def __init__(self, device="cpu", seed: int = 0, dtype=torch.float32):
        self.device, self.dtype = torch.device(device), dtype
        self.nodes: List[_Node] = []
        self._params: Dict[str, FTensor] = {}
        self._modules: Dict[str, FModule] = {}
        self._grad_on = True
        self.gen = torch.Generator(device=self.device).manual_seed(seed)

    # ---- leaves
    def param(self, rows: int, cols: int, init: str = "kaiming", name: str = None, decay: bool = True) -> FTensor:
        """A trainable [rows, cols] matrix that persists across ``reset``.  ``init``: kaiming (fan-in = rows), xavier, zeros,
        ones, or normal."""
        name = name or f"p{len(self._params)}"
        if name in self._params:
            raise KeyError(f"parameter {name!r} exists")
        p = Param(name, (rows, cols), decay=decay, device=self.device, pad_rows=False)
        g = torch.Generator().manual_seed(zlib.crc32(name.encode()) + int(self.gen.initial_seed()))
        if init in ("kaiming", "xavier", "normal"):
            std = {"kaiming": math.sqrt(2.0 / rows), "xavier": math.sqrt(2.0 / (rows + cols)), "normal": 1.0}[init]
            p.data.copy_(torch.randn(rows, cols, generator=g) * std)
        elif init == "ones":
            p.data.fill_(1.0)
        elif init != "zeros":
            raise ValueError(init)
        t = FTensor(self, _Node("param", (), None, param=p))
        self._params[name] = t
        return t

    def zeros(self, rows: int, cols: int, name: str = None) -> FTensor:
        return self.param(rows, cols, "zeros", name, decay=False)

    def constant(self, data) -> FTensor:
        v = data if isinstance(data, torch.Tensor) else torch.as_tensor(data, dtype=self.dtype)
        return FTensor(self, _Node("const", (), v.to(self.device, self.dtype), needs_grad=False))

    def input(self, data) -> FTensor:
        """A leaf that receives a gradient (read it from ``.grad`` after ``backward``)."""
        t = self.constant(data)
        t.node.needs_grad = True
        t.node.op = "input"
        if self._grad_on:
            self.nodes.append(t.node)
        return t

    def module(self, mod, name: str) -> FModule:
        if name in self._modules:
            raise KeyError(f"module {name!r} exists")
        self._modules[name] = FModule(self, mod.to(self.device) if hasattr(mod, "to") else mod, name)
        return self._modules[name]

    # ---- what nn's optimizers and checkpoint writers walk
    def named_params(self) -> Iterator[Tuple[str, Param]]:
        for name, t in self._params.items():
            yield name, t.node.param
        for mname, fm in self._modules.items():
            for name, p in fm.module.named_params():
                yield f"{mname}.{name}", p

    def zero_grad(self):
        for _, p in self.named_params():
            if p._grd is not None:
                p._grd.zero_()

    # ---- recording
    @contextlib.contextmanager
    def no_grad(self):
        old, self._grad_on = self._grad_on, False
        try:
            yield self
        finally:
            self._grad_on = old

    def reset(self):
        """Drop the nodes of the step; parameters and modules stay."""
        self.nodes.clear()

    def _record(self, op, inputs, value, saved=None, force: bool = False) -> FTensor:
        """``force``: the node holds parameters of its own (a module), so it is recorded even on constant inputs."""
        needs = self._grad_on and (force or any(i.node.needs_grad for i in inputs))
        node = _Node(op, tuple(i.node for i in inputs), value, saved if needs else None, needs_grad=needs)
        if needs:
            self.nodes.append(node)
        return FTensor(self, node)

    # ---- reverse pass
    def backward(self, out: FTensor, seed: torch.Tensor = None):
        for n in self.nodes:
            n.grad = None
        out.node.grad = torch.ones_like(out.node.value) if seed is None else seed.to(out.node.value)
        for n in reversed(self.nodes):
            if n.grad is None or n.op in ("input",):
                continue
            _BACKWARD[n.op](n)

    def __len__(self):
        return len(self.nodes)


def _acc(n: _Node, g: torch.Tensor):
    if not n.needs_grad:
        return
    g = _unbroadcast(g, n.v.shape)
    if n.param is not None:
        if not n.param.frozen:
            n.param.grad.add_(g)
    elif n.grad is None:
        n.grad = g
    else:
        n.grad = n.grad + g


def _bw_add(n):
    _acc(n.inputs[0], n.grad), _acc(n.inputs[1], n.grad)


def _bw_sub(n):
    _acc(n.inputs[0], n.grad), _acc(n.inputs[1], -n.grad)


def _bw_mul(n):
    a, b = n.inputs
    _acc(a, n.grad * b.v), _acc(b, n.grad * a.v)


def _bw_div(n):
    a, b = n.inputs
    _acc(a, n.grad / b.v), _acc(b, -n.grad * a.v / (b.v * b.v))


def _bw_matmul(n):
    a, b = n.inputs
    g = n.grad
    if a.v.dim() == 2 and b.v.dim() == 2:
        if a.needs_grad:
            _acc(a, _mm_nt(g.contiguous(), b.v))
        if b.needs_grad:
            _acc(b, _mm_tn(a.v, g.contiguous()))
    else:
        _acc(a, g @ b.v.transpose(-1, -2)), _acc(b, a.v.transpose(-1, -2) @ g)


def _expand_reduced(g, axis, keepdim, shape):
    if axis is None:
        return g.expand(shape)
    if not keepdim:
        g = g.unsqueeze(axis) if isinstance(axis, int) else g.reshape([1 if i in [a % len(shape) for a in axis] else s for i, s in enumerate(shape)])
    return g.expand(shape)


def _bw_sum(n):
    axis, keepdim, shape = n.saved
    _acc(n.inputs[0], _expand_reduced(n.grad, axis, keepdim, shape))


def _bw_mean(n):
    axis, keepdim, shape = n.saved
    full = _expand_reduced(n.grad, axis, keepdim, shape)
    _acc(n.inputs[0], full * (n.value.numel() / max(1, math.prod(shape))))


def _bw_max(n):
    axis, keepdim, idx, shape = n.saved
    g = n.grad if keepdim else n.grad.unsqueeze(axis)
    _acc(n.inputs[0], torch.zeros(shape, device=g.device, dtype=g.dtype).scatter_(axis, idx, g))


def _bw_narrow(n):
    dim, start, length, shape = n.saved
    full = torch.zeros(shape, device=n.grad.device, dtype=n.grad.dtype)
    full.narrow(dim, start, length).copy_(n.grad)
    _acc(n.inputs[0], full)


def _bw_act(n):
    x, name = n.inputs[0].v, n.saved
    d = _gelu_grad(x) if name == "gelu" else _ACT[name][1](x, n.value)
    _acc(n.inputs[0], n.grad * d)


def _bw_softmax(n):
    y, ax = n.value, n.saved
    _acc(n.inputs[0], y * (n.grad - (n.grad * y).sum(ax, keepdim=True)))


def _bw_log_softmax(n):
    ax = n.saved
    _acc(n.inputs[0], n.grad - torch.exp(n.value) * n.grad.sum(ax, keepdim=True))


def _bw_clamp(n):
    lo, hi = n.saved
    x = n.inputs[0].v
    m = torch.ones_like(x, dtype=torch.bool)
    if lo is not None:
        m &= x >= lo
    if hi is not None:
        m &= x <= hi
    _acc(n.inputs[0], n.grad * m)


def _bw_linear(n):
    x, w, b = n.inputs
    act, pre = n.saved
    g = n.grad
    if act is not None:
        g = g * (_gelu_grad(pre) if act == "gelu" else _ACT[act][1](pre, n.value))
    g = g.contiguous()
    if w.needs_grad:
        _acc(w, _mm_tn(x.v, g))
    if b is not None and b.needs_grad:
        _acc(b, g.sum(0, keepdim=True))
    if x.needs_grad:
        _acc(x, _mm_nt(g, w.v))


def _bw_cross_entropy(n):
    logp, target = n.saved
    g = torch.exp(logp)
    g.scatter_add_(1, target[:, None], -torch.ones_like(g[:, :1]))
    _acc(n.inputs[0], g * (n.grad / logp.shape[0]))


def _bw_concat(n):
    axis, sizes = n.saved
    for i, piece in zip(n.inputs, torch.split(n.grad, sizes, axis)):
        _acc(i, piece)


def _bw_gather(n):
    axis, idx, shape = n.saved
    _acc(n.inputs[0], torch.zeros(shape, device=n.grad.device, dtype=n.grad.dtype).scatter_add_(axis, idx, n.grad))


def _bw_module(n):
    mod = n.saved
    dx = mod.vjp(n.grad.to(torch.bfloat16).contiguous() if n.grad.is_cuda else n.grad)
    dxs = dx if isinstance(dx, (tuple, list)) else (dx,)
    for i, d in zip(n.inputs, dxs):
        if d is not None:
            _acc(i, d.float())


_BACKWARD = {
    "add": _bw_add, "sub": _bw_sub, "mul": _bw_mul, "div": _bw_div, "matmul": _bw_matmul,
    "neg": lambda n: _acc(n.inputs[0], -n.grad),
    "pow": lambda n: _acc(n.inputs[0], n.grad * n.saved * n.inputs[0].v ** (n.saved - 1)),
    "transpose": lambda n: _acc(n.inputs[0], n.grad.transpose(*n.saved)),
    "permute": lambda n: _acc(n.inputs[0], n.grad.permute(*torch.argsort(torch.tensor(n.saved)).tolist())),
    "reshape": lambda n: _acc(n.inputs[0], n.grad.reshape(n.saved)),
    "narrow": _bw_narrow, "sum": _bw_sum, "mean": _bw_mean, "max": _bw_max,
    "exp": lambda n: _acc(n.inputs[0], n.grad * n.value),
    "log": lambda n: _acc(n.inputs[0], n.grad / n.inputs[0].v),
    "sqrt": lambda n: _acc(n.inputs[0], n.grad * 0.5 / n.value),
    "clamp": _bw_clamp, "act": _bw_act, "softmax": _bw_softmax, "log_softmax": _bw_log_softmax,
    "dropout": lambda n: _acc(n.inputs[0], n.grad * n.saved),
    "linear": _bw_linear, "cross_entropy": _bw_cross_entropy, "concat": _bw_concat, "gather": _bw_gather, "module": _bw_module,
}


class F:
    """Fused and composite operations."""

    @staticmethod
    def linear(x: FTensor, w: FTensor, b: FTensor = None, act: str = None) -> FTensor:
        """``act(x @ w + b)`` as ONE node: w is [in, out], b [1, out]."""
        xv, wv = x.value, w.value
        if _use_gemm(xv, wv) and act in (None, "relu", "tanh", "sigmoid"):
            from .. import ops
            y = ops.gemm(xv, wv, b_mn=True, bias=b.value.reshape(-1) if b is not None else None, act=act)
            pre = None                                          # these derivatives read the output
        else:
            pre = xv @ wv
            if b is not None:
                pre = pre + b.value
            y = pre if act is None else _ACT[act][0](pre)
        ins = (x, w) if b is None else (x, w, b)
        t = x.tape._record("linear", ins, y, saved=(act, pre))
        if b is None:
            t.node.inputs = (x.node, w.node, None)
        return t

    @staticmethod
    def mse(pred: FTensor, target) -> FTensor:
        d = pred - target
        return (d * d).mean()

    @staticmethod
    def cross_entropy(logits: FTensor, target: torch.Tensor) -> FTensor:
        """Mean negative log-likelihood of integer targets, fused: one node, gradient softmax − one-hot."""
        logp = torch.log_softmax(logits.value, -1)
        tgt = target.to(logits.value.device).long()
        v = -logp.gather(1, tgt[:, None]).mean()
        return logits.tape._record("cross_entropy", (logits,), v, saved=(logp, tgt))

    @staticmethod
    def dropout(x: FTensor, p: float, training: bool = True) -> FTensor:
        """Seeded by the tape's generator: the same tape seed gives the same masks."""
        if not training or p <= 0:
            return x
        keep = (torch.rand(x.shape, device=x.tape.device, generator=x.tape.gen) >= p).float() / (1 - p)
        return x.tape._record("dropout", (x,), x.value * keep, saved=keep)

    @staticmethod
    def concat(xs: Sequence[FTensor], axis: int = 0) -> FTensor:
        return xs[0].tape._record("concat", tuple(xs), torch.cat([x.value for x in xs], axis),
                                  saved=(axis, [x.shape[axis] for x in xs]))

    @staticmethod
    def gather(x: FTensor, axis: int, index: torch.Tensor) -> FTensor:
        idx = index.to(x.tape.device).long()
        return x.tape._record("gather", (x,), x.value.gather(axis, idx), saved=(axis, idx, x.shape))

    @staticmethod
    def layer_norm(x: FTensor, gamma: FTensor = None, beta: FTensor = None, eps: float = 1e-5) -> FTensor:
        """Composite of tape operations (mean, variance, scale, shift)."""
        mu = x.mean(-1, keepdim=True)
        c = x - mu
        y = c / ((c * c).mean(-1, keepdim=True) + eps).sqrt()
        if gamma is not None:
            y = y * gamma
        return y + beta if beta is not None else y


class TapeAdam:
    """Adam over the tape's parameters (and those of its modules) through the arena optimizer of ``nn``.  Build it after the
    last parameter: the arena is laid out once."""

    def __init__(self, tape: Tape, lr: float = 1e-3, **kw):
        from ..nn.optim import Adam
        self.tape, self.opt = tape, Adam(list(tape.named_params()), lr=lr, device=tape.device, **kw)

    def step(self):
        self.opt.step()
        self.opt.zero_grad()
