"""Leaf modules, part 1: dense layers and activations.

``Linear`` stores its weight ``[IN, OUT]`` row-major — the transpose of torch's ``[out, in]`` —
exactly like the reference (noeira/nn/primitives/linear.mojo:970-971, torch_names.mojo:11-16), so
forward, dgrad and wgrad are the NN / NT / TN cases of one tcgen05 GEMM and no transposed copy of the
weight exists anywhere.  Parameter names: ``weight`` (decay), ``bias`` (no decay).
"""
from __future__ import annotations

import ctypes

import torch

from .. import ops
from .._native import check, cuda_lib, ptr, stream_ptr
from .init import Constant, Initializer, Kaiming, Zero
from .module import Module

_ACT_CPU = {
    None: (lambda x: x), "none": (lambda x: x), "relu": torch.relu, "tanh": torch.tanh,
    "gelu": (lambda x: torch.nn.functional.gelu(x, approximate="tanh")), "silu": torch.nn.functional.silu,
    "sigmoid": torch.sigmoid,
}
# which tensor the derivative is evaluated on: the output (cheap to keep) or the input
SAVES_OUTPUT = {"relu", "tanh", "sigmoid"}


def act_derivative_cpu(act, saved):
    if act in (None, "none"):
        return torch.ones_like(saved)
    if act == "relu":
        return (saved > 0).to(saved.dtype)
    if act == "tanh":
        return 1 - saved * saved
    if act == "sigmoid":
        return saved * (1 - saved)
    x = saved.detach().clone().requires_grad_(True)
    with torch.enable_grad():
        _ACT_CPU[act](x).sum().backward()
    return x.grad


def act_backward(dy, saved, act):
    """dx = dy ⊙ f'(saved) (bf16 kernel on CUDA, torch on CPU)."""
    if act in (None, "none"):
        return dy
    if dy.is_cuda:
        dy = dy.contiguous()
        saved = saved.contiguous()
        dx = torch.empty_like(dy)
        check(cuda_lib().nb_act_bwd(ptr(dy), ptr(saved), ptr(dx), ctypes.c_longlong(dy.numel()),
                                    ctypes.c_int(_act_code(act)),
                                    stream_ptr()), "act_bwd")
        return dx
    return dy * act_derivative_cpu(act, saved)


def _act_code(act):
    from ..ops.gemm import ACT
    return ACT[act]


_COLSUM_WS = {}


def _colsum_workspace(device, need: int):
    from ..ops.streams import ws_key
    key = ws_key(device)
    ws = _COLSUM_WS.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.empty(max(need, 256 * 8192), dtype=torch.float32, device=device)
        _COLSUM_WS[key] = ws
    return ws


def colsum_into(dy, out_f32, n, accumulate=True):
    """out[:n] (+)= Σ_rows dy[:, :n]  (two-stage, deterministic)."""
    if dy.is_cuda:
        lib = cuda_lib()
        split = lib.nb_colsum_split(ctypes.c_int(dy.shape[0]))
        ws = _colsum_workspace(dy.device, split * n)
        check(lib.nb_colsum_bf16(ptr(dy), ctypes.c_int(dy.shape[0]), ctypes.c_int(n), ctypes.c_int(dy.stride(0)),
                                 ptr(out_f32), ctypes.c_int(int(accumulate)), ptr(ws), stream_ptr()), "colsum")
    else:
        s = dy[:, :n].float().sum(0)
        if accumulate:
            out_f32[:n] += s
        else:
            out_f32[:n] = s


class Linear(Module):
    """y = act(x @ W + b).  ``act`` fused in the GEMM epilogue (``LinearAct`` of the reference,
    noeira/nn/primitives/linear_act.mojo; cuBLASLt EPI_* there, tcgen05 epilogue functors here)."""

    def __init__(self, in_dim: int, out_dim: int, act: str = None, bias: bool = True, init: Initializer = None,
                 out_fp32: bool = False, need_input_grad: bool = True):
        super().__init__()
        self.in_dim, self.out_dim, self.act = int(in_dim), int(out_dim), (None if act in (None, "none") else act)
        self.weight = self.add_param("weight", (in_dim, out_dim), decay=True, init=init or Kaiming(), fan_in=in_dim,
                                     fan_out=out_dim)
        self.bias = self.add_param("bias", (out_dim,), decay=False, init=Zero()) if bias else None
        self.out_fp32 = out_fp32
        self.need_input_grad = need_input_grad
        self._x = self._saved = None

    def display_label(self):
        return f"Linear[{self.in_dim},{self.out_dim}]" + (f"+{self.act}" if self.act else "")

    @property
    def out_pad(self):
        return self.weight.storage_shape[1]

    # ---- forward
    def forward(self, x, residual=None):
        """``residual`` (same shape as the output) is added to the result; on CUDA the addition happens in the GEMM
        epilogue when the layer has no activation.  Its gradient is the caller's business (identity)."""
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        self._lead = lead
        self._x = x2
        if not self.on_cuda:
            pre = x2[:, : self.in_dim].float() @ self.weight.data
            if self.bias is not None:
                pre = pre + self.bias.data
            y = _ACT_CPU[self.act](pre)
            self._saved = y if self.act in SAVES_OUTPUT else pre
            y = y.reshape(*lead, self.out_dim)
            return y if residual is None else y + residual
        if self.attrs.get("precision") == "tf32":
            return self._forward_tf32(x2, lead, residual)
        W = self.weight.shadow
        b = self.bias.storage if self.bias is not None else None
        xa = x2[:, : self.in_dim]
        res = None
        if residual is not None and self.act is None and not self.out_fp32 and self.out_pad == self.out_dim:
            res = residual.reshape(-1, self.out_dim)
            if res.dtype != torch.bfloat16 or res.stride(-1) != 1 or res.stride(0) % 8:
                res = None
        if self.act is None or self.act in SAVES_OUTPUT or not torch.is_grad_enabled():
            # no backward will follow under no_grad: any activation can then be fused, nothing needs saving
            y = ops.gemm(xa, W, b_mn=True, bias=b, act=self.act, residual=res,
                         out_dtype=torch.float32 if self.out_fp32 else torch.bfloat16)
            self._saved = y if res is None else None
            if res is not None:
                residual = None
        else:
            pre = ops.gemm(xa, W, b_mn=True, bias=b)
            y = torch.empty_like(pre)
            check(cuda_lib().nb_act_fwd(ptr(pre), ptr(y), ctypes.c_longlong(pre.numel()), ctypes.c_int(_act_code(self.act)),
                                        stream_ptr()), "act_fwd")
            self._saved = pre
        if self.out_pad != self.out_dim:
            y = y[:, : self.out_dim]
        y = y.reshape(*lead, self.out_dim) if len(lead) != 1 else y
        return y if residual is None else y + residual

    # ---- backward
    def vjp(self, dy, dy_is_pre: bool = False, fuse_dact=None):
        """``fuse_dact=(act, saved)`` folds the PREVIOUS layer's activation derivative into this layer's
        dgrad epilogue; the caller then passes ``dy_is_pre=True`` to that layer."""
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not self.on_cuda:
            dpre = dy2.float()
            if self.act is not None and not dy_is_pre:
                dpre = dpre * act_derivative_cpu(self.act, self._saved)
            x = self._x[:, : self.in_dim].float()
            if not self.weight.frozen:
                self.weight.grad.add_(x.t() @ dpre)
                if self.bias is not None:
                    self.bias.grad.add_(dpre.sum(0))
            if not self.need_input_grad:
                return None
            dx = dpre @ self.weight.data.t()
            if fuse_dact is not None:
                dx = dx * act_derivative_cpu(fuse_dact[0], fuse_dact[1].reshape(dx.shape[0], -1)[:, : self.in_dim].float())
            return dx.reshape(*self._lead, self.in_dim)
        if self.attrs.get("precision") == "tf32":
            return self._vjp_tf32(dy2, dy_is_pre, fuse_dact)
        if dy2.dtype != torch.bfloat16:
            dy2 = dy2.to(torch.bfloat16)
        if dy2.stride(-1) != 1 or (dy2.stride(0) * 2) % 16 != 0 or dy2.data_ptr() % 16 != 0:
            dy2 = _pad_rows(dy2)
        if self.act is not None and not dy_is_pre:
            sv = self._saved if self._saved.dtype == torch.bfloat16 else self._saved.to(torch.bfloat16)
            dy2 = act_backward(dy2.contiguous(), sv[:, : dy2.shape[1]].contiguous() if sv.shape[1] != dy2.shape[1] else sv, self.act)
            if (dy2.stride(0) * 2) % 16 != 0:           # narrow outputs (e.g. 6 actions): back to a 16-byte row pitch
                dy2 = _pad_rows(dy2)
        n = self.out_dim
        dyv = dy2[:, :n]
        if not self.weight.frozen:
            br = self.attrs.get("grad_branch")
            if br is not None:
                # parameter gradients leave the critical path: they run on the branch's stream while the data
                # gradient continues here; the owner joins the branch before its optimizer step
                with br:
                    self._param_grads(dy2, dyv, n)
                br.keep(dy2, self._x)
            else:
                self._param_grads(dy2, dyv, n)
        if not self.need_input_grad:
            return None
        W = self.weight.shadow
        in_pad = (self.in_dim + 7) // 8 * 8
        alloc = torch.empty if in_pad == self.in_dim else torch.zeros
        dx = alloc(dy2.shape[0], in_pad, device=dy2.device, dtype=torch.bfloat16)
        aux, dact = (None, None)
        if fuse_dact is not None:
            dact, aux = fuse_dact
            aux = aux.reshape(dy2.shape[0], -1)
        ops.gemm(dyv, W[:, :n], out=dx, aux=aux, dact=dact, n=self.in_dim)
        dx = dx[:, : self.in_dim] if in_pad != self.in_dim else dx
        return dx.reshape(*self._lead, self.in_dim) if len(self._lead) != 1 else dx

    # ---- fp32 activations on the TF32 tensor-core path (``set_attr("precision", "tf32")``): the fp32 master weights are
    # the operands, no bf16 shadow is read; activations, saved tensors and gradients stay fp32
    @staticmethod
    def _rows4(t):
        """fp32 [M, n] with a 16-byte aligned base and row pitch (TMA): a padded copy only when needed."""
        if t.dtype == torch.float32 and t.stride(-1) == 1 and t.stride(0) % 4 == 0 and t.data_ptr() % 16 == 0:
            return t
        out = torch.zeros(t.shape[0], (t.shape[1] + 3) // 4 * 4, device=t.device, dtype=torch.float32)
        out[:, : t.shape[1]] = t
        return out[:, : t.shape[1]]

    def _forward_tf32(self, x2, lead, residual):
        xa = self._rows4(x2[:, : self.in_dim])
        self._x = xa
        b = self.bias.storage if self.bias is not None else None
        fuse = self.act is None or self.act in SAVES_OUTPUT or not torch.is_grad_enabled()
        y = ops.gemm(xa, self.weight.storage, b_mn=True, bias=b, act=self.act if fuse else None)
        if fuse:
            self._saved = y
        else:
            self._saved = y
            y = _ACT_CPU[self.act](y)
        if self.out_pad != self.out_dim:
            y = y[:, : self.out_dim]
        y = y.reshape(*lead, self.out_dim) if len(lead) != 1 else y
        return y if residual is None else y + residual

    def _vjp_tf32(self, dy2, dy_is_pre, fuse_dact):
        n = self.out_dim
        d = dy2[:, :n].float()
        if self.act is not None and not dy_is_pre:
            d = d * act_derivative_cpu(self.act, self._saved[:, :n])
        d = self._rows4(d)
        if not self.weight.frozen:
            ops.gemm(self._x, d, a_mn=True, b_mn=True, out=self.weight.grad_storage, accumulate=True, n=n)
            if self.bias is not None:
                self.bias.grad_storage[:n].add_(d.sum(0))
        if not self.need_input_grad:
            return None
        in4 = (self.in_dim + 3) // 4 * 4
        dx = (torch.empty if in4 == self.in_dim else torch.zeros)(d.shape[0], in4, device=d.device, dtype=torch.float32)
        ops.gemm(d, self.weight.storage[:, :n], out=dx, n=self.in_dim)
        dx = dx[:, : self.in_dim]
        if fuse_dact is not None:
            dx = dx * act_derivative_cpu(fuse_dact[0], fuse_dact[1].reshape(dx.shape[0], -1)[:, : self.in_dim].float())
        return dx.reshape(*self._lead, self.in_dim) if len(self._lead) != 1 else dx

    def _param_grads(self, dy2, dyv, n):
        ops.gemm(self._x[:, : self.in_dim], dyv, a_mn=True, b_mn=True, out=self.weight.grad_storage, accumulate=True, n=n)
        if self.bias is not None:
            colsum_into(dy2, self.bias.grad_storage, n)

    def _release(self):
        self._x = self._saved = None


def _pad_rows(t):
    """Copy into a tensor whose row pitch is a multiple of 8 elements (16 bytes in bf16)."""
    p = (t.shape[1] + 7) // 8 * 8
    out = torch.zeros(t.shape[0], p, device=t.device, dtype=t.dtype)
    out[:, : t.shape[1]] = t
    return out[:, : t.shape[1]]


def LinearReLU(i, o, **kw):
    return Linear(i, o, act="relu", **kw)


def LinearTanh(i, o, **kw):
    return Linear(i, o, act="tanh", **kw)


def LinearGELU(i, o, **kw):
    return Linear(i, o, act="gelu", **kw)


class Elementwise(Module):
    """Standalone activation (noeira/nn/primitives/elementwise.mojo)."""

    def __init__(self, act: str):
        super().__init__()
        self.act = act

    def forward(self, x):
        if not x.is_cuda:
            y = _ACT_CPU[self.act](x.float())
            self._saved = y if self.act in SAVES_OUTPUT else x.float()
            return y
        xc = x.contiguous()
        y = torch.empty_like(xc)
        check(cuda_lib().nb_act_fwd(ptr(xc), ptr(y), ctypes.c_longlong(xc.numel()), ctypes.c_int(_act_code(self.act)),
                                    stream_ptr()), "act_fwd")
        self._saved = y if self.act in SAVES_OUTPUT else xc
        return y

    def vjp(self, dy):
        return act_backward(dy if not dy.is_cuda else dy.contiguous(), self._saved, self.act)


class GaussianHead(Module):
    """μ = Linear(H → ACT) plus ONE learnable state-independent ln σ vector
    (noeira/deep_agents/primitives/gaussian_head.mojo:1-136).  ``forward`` returns μ in fp32
    (``[M, ACT]``); ``packed()`` gives the reference's ``[μ | ln σ]`` layout."""

    LS_MIN, LS_MAX = -5.0, 2.0

    def __init__(self, hidden: int, act_dim: int, log_std_init: float = -0.5, init: Initializer = None):
        super().__init__()
        self.act_dim = act_dim
        self.lin = Linear(hidden, act_dim, out_fp32=True, init=init)
        # the reference exposes weight / bias / log_std directly on the head
        self._params["weight"] = self.lin.weight
        self._params["bias"] = self.lin.bias
        self.log_std = self.add_param("log_std", (act_dim,), decay=False, init=Constant(log_std_init))

    def _moved(self, device):
        self.lin.device = device

    def _attr_changed(self, name, value):
        self.lin.attrs[name] = value            # the inner layer is not a registered child (its parameters are exposed here)
        if name == "training":
            self.lin.training = bool(value)

    def forward(self, x):
        self._mu = self.lin.forward(x)
        return self._mu

    def packed(self):
        ls = self.log_std.data.clamp(self.LS_MIN, self.LS_MAX)
        return torch.cat([self._mu.float(), ls.expand(self._mu.shape[0], -1)], dim=1)

    def vjp(self, dmu, fuse_dact=None):
        return self.lin.vjp(dmu, fuse_dact=fuse_dact)

    def _release(self):
        self.lin._release()


class BiasAdd(Module):
    def __init__(self, dim):
        super().__init__()
        self.bias = self.add_param("bias", (dim,), decay=False, init=Zero())

    def forward(self, x):
        return x + self.bias.data.to(x.dtype)

    def vjp(self, dy):
        self.bias.grad.add_(dy.reshape(-1, dy.shape[-1]).float().sum(0))
        return dy


class Scale(Module):
    def __init__(self, multiplier: float = 1.0):
        super().__init__()
        self.multiplier = multiplier

    def _attr_changed(self, name, value):
        if name == "multiplier":
            self.multiplier = float(value)

    def forward(self, x):
        return x * self.multiplier

    def vjp(self, dy):
        return dy * self.multiplier


_RNG_STEP = {}
_DROPOUT_IDS = [0]


def rng_step_counter(device) -> torch.Tensor:
    """Device-resident step counter (uint64 in an int64 tensor) that every counter-hash random op reads."""
    key = torch.device(device).index or 0
    t = _RNG_STEP.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int64, device=device)
        _RNG_STEP[key] = t
    return t


def advance_rng(device, inc: int = 1):
    """counter += inc, as a kernel on the current stream: call once per training step (inside a captured step)."""
    if torch.device(device).type != "cuda":
        return
    check(cuda_lib().nb_u64_add(ptr(rng_step_counter(device)), ctypes.c_ulonglong(inc), stream_ptr()), "u64_add")


class Dropout(Module):
    """Counter-hash dropout: the mask is a pure function of (module seed, step counter, element index), so a
    captured graph replays fresh masks (noeira/nn/random/hash_mask.mojo).  On CUDA the counter lives on the
    device (``advance_rng``); on CPU a host counter seeds a generator."""

    def __init__(self, p: float = 0.1, seed: int = 0):
        super().__init__()
        _DROPOUT_IDS[0] += 1
        self.p, self.seed, self.counter = p, seed * 1000003 + _DROPOUT_IDS[0] * 7919, 0

    def forward(self, x):
        if not self.training or self.p == 0.0:
            self._mask = None
            return x
        if x.is_cuda:
            xc = x if (x.is_contiguous() and x.dtype == torch.bfloat16) else x.to(torch.bfloat16).contiguous()
            y = torch.empty_like(xc)
            self._mask = torch.empty(xc.numel() + 8, dtype=torch.uint8, device=x.device)
            check(cuda_lib().nb_dropout_fwd(ptr(xc), ptr(y), ptr(self._mask), ctypes.c_longlong(xc.numel()),
                                            ctypes.c_ulonglong(self.seed), ptr(rng_step_counter(x.device)),
                                            ctypes.c_float(self.p), stream_ptr()), "dropout_fwd")
            return y
        g = torch.Generator(device=x.device).manual_seed(self.seed + self.counter)
        self.counter += 1
        self._mask = (torch.rand(x.shape, device=x.device, generator=g) >= self.p).to(x.dtype) / (1.0 - self.p)
        return x * self._mask

    def vjp(self, dy):
        if self._mask is None:
            return dy
        if dy.is_cuda:
            d = dy if (dy.is_contiguous() and dy.dtype == torch.bfloat16) else dy.to(torch.bfloat16).contiguous()
            dx = torch.empty_like(d)
            check(cuda_lib().nb_dropout_bwd(ptr(d), ptr(self._mask), ptr(dx), ctypes.c_longlong(d.numel()),
                                            ctypes.c_float(self.p), stream_ptr()), "dropout_bwd")
            return dx
        return dy * self._mask
