"""Linear layers with structure: factorised-noise weights and block-diagonal ensembles.

``NoisyLinear``: ``y = x μ_w + ((x ⊙ f(ε_in)) σ_w) ⊙ f(ε_out) + μ_b + σ_b ⊙ f(ε_out)`` with ``f(e) = sign(e) √|e|`` and
independent standard-normal ``ε_in [in]``, ``ε_out [out]`` (factorised Gaussian noise).  The effective weight
``μ_w + σ_w ⊙ (f_in ⊗ f_out)`` is never materialised: the layer is two GEMMs on the same input, the second on the
input scaled by ``f_in`` with its output scaled by ``f_out``; the backward reuses the same split, so the gradients of
``σ_w`` and ``σ_b`` are ordinary weight / bias gradients of the second GEMM.  ``reset_noise`` redraws the factors on the
device; in eval mode the layer is its mean.  Parameter names ``mu_w, sigma_w, mu_b, sigma_b``
(noeira/nn/primitives/noisy_linear.mojo: materialised effective weight and factorised gradient kernels there).

``BlockLinear``: ``BLOCKS`` independent ``in → out`` maps evaluated as one batched contraction on ``[B, BLOCKS, in]``
(ensembles of critics or dynamics models in one call; noeira/nn/primitives/block_linear.mojo).
"""
from __future__ import annotations

import math

import torch

from .init import Constant, Initializer, Kaiming
from .layers import _ACT_CPU, SAVES_OUTPUT, Linear, act_derivative_cpu
from .module import Module


def _f(e):
    return e.sign() * e.abs().sqrt()


class NoisyLinear(Module):
    def __init__(self, in_dim: int, out_dim: int, sigma0: float = 0.5, out_fp32: bool = False, need_input_grad: bool = True):
        super().__init__()
        self.in_dim, self.out_dim = int(in_dim), int(out_dim)
        s = sigma0 / math.sqrt(in_dim)
        self.mu = self.add_child("mu", Linear(in_dim, out_dim, out_fp32=True, need_input_grad=need_input_grad))
        self.sigma = self.add_child("sigma", Linear(in_dim, out_dim, init=Constant(s), out_fp32=True, need_input_grad=need_input_grad))
        self.sigma.bias.set_(torch.full((out_dim,), s))
        self.out_fp32 = out_fp32
        self.need_input_grad = need_input_grad
        self.f_in = torch.zeros(in_dim)
        self.f_out = torch.zeros(out_dim)
        self._noisy = False

    # the two GEMMs are children for device moves / release, but their parameters carry the layer's own names
    def named_params(self, prefix: str = ""):
        yield prefix + "mu_w", self.mu.weight
        yield prefix + "sigma_w", self.sigma.weight
        yield prefix + "mu_b", self.mu.bias
        yield prefix + "sigma_b", self.sigma.bias

    def _moved(self, device):
        self.f_in, self.f_out = self.f_in.to(device), self.f_out.to(device)

    def display_label(self):
        return f"NoisyLinear[{self.in_dim},{self.out_dim}]"

    def reset_noise(self, generator: torch.Generator = None):
        """Redraw the noise factors (on the layer's device; the tensors keep their addresses, so a captured step sees the
        new values)."""
        dev = self.f_in.device
        self.f_in.copy_(_f(torch.randn(self.in_dim, device=dev, generator=generator)))
        self.f_out.copy_(_f(torch.randn(self.out_dim, device=dev, generator=generator)))

    def forward(self, x):
        self._noisy = self.training
        y = self.mu.forward(x).float()
        if self._noisy:
            xs = x * self.f_in.to(x.dtype)
            y = y + self.sigma.forward(xs).float() * self.f_out
        return y if self.out_fp32 or not x.is_cuda else y.to(torch.bfloat16)

    def vjp(self, dy):
        dy = dy.float()
        dx = self.mu.vjp(dy)
        if self._noisy:
            dxs = self.sigma.vjp(dy * self.f_out)
            if dx is not None:
                dx = dx + dxs * self.f_in.to(dxs.dtype)
        return dx


def reset_noise(module: Module, generator: torch.Generator = None):
    """Redraw the noise of every ``NoisyLinear`` under ``module``."""
    for m in module.modules():
        if isinstance(m, NoisyLinear):
            m.reset_noise(generator)


class _BlockInit(Initializer):
    def __call__(self, shape, fan_in, fan_out, gen):
        return Kaiming()(shape, fan_in, fan_out, gen)


class BlockLinear(Module):
    """``y[b, k] = act(x[b, k] @ W[k] + bias[k])`` for k < BLOCKS; input ``[B, BLOCKS, in]`` (or ``[B, in]``, shared by every
    block), output ``[B, BLOCKS, out]``.  One batched contraction per direction."""

    def __init__(self, in_dim: int, out_dim: int, blocks: int, act: str = None, need_input_grad: bool = True):
        super().__init__()
        self.in_dim, self.out_dim, self.blocks = int(in_dim), int(out_dim), int(blocks)
        self.act = None if act in (None, "none") else act
        self.weight = self.add_param("weight", (blocks * in_dim, out_dim), decay=True, init=_BlockInit(), fan_in=in_dim,
                                     fan_out=out_dim)
        self.bias = self.add_param("bias", (blocks * out_dim,), decay=False, init=Constant(0.0))
        self.need_input_grad = need_input_grad
        self._x = self._saved = None
        self._shared = False

    def display_label(self):
        return f"BlockLinear[{self.blocks}x{self.in_dim},{self.out_dim}]" + (f"+{self.act}" if self.act else "")

    def _w(self):
        w = self.weight.data if not self.on_cuda else self.weight.shadow[:, : self.out_dim]
        return w.reshape(self.blocks, self.in_dim, -1)[..., : self.out_dim]

    def forward(self, x):
        self._shared = x.dim() == 2
        xb = x[:, None, :].expand(-1, self.blocks, -1) if self._shared else x
        self._x = xb
        w = self._w()
        bias = (self.bias.data if not self.on_cuda else self.bias.storage[: self.blocks * self.out_dim]).reshape(self.blocks, self.out_dim)
        pre = torch.einsum("bki,kio->bko", xb.to(w.dtype), w).float() + bias.float()
        y = _ACT_CPU[self.act](pre)
        self._saved = y if self.act in SAVES_OUTPUT else pre
        return y if not x.is_cuda else y.to(torch.bfloat16)

    def vjp(self, dy):
        dpre = dy.float()
        if self.act is not None:
            dpre = dpre * act_derivative_cpu(self.act, self._saved)
        x = self._x.float()
        gw = torch.einsum("bki,bko->kio", x, dpre).reshape(self.blocks * self.in_dim, self.out_dim)
        gb = dpre.sum(0).reshape(-1)
        if not self.weight.frozen:
            if self.on_cuda:
                self.weight.grad_storage.reshape(self.blocks * self.in_dim, -1)[:, : self.out_dim].add_(gw)
                self.bias.grad_storage[: gb.numel()].add_(gb)
            else:
                self.weight.grad.add_(gw)
                self.bias.grad.add_(gb)
        if not self.need_input_grad:
            return None
        dx = torch.einsum("bko,kio->bki", dpre, self._w().float())
        if self._shared:
            dx = dx.sum(1)
        return dx if not dy.is_cuda else dx.to(torch.bfloat16)

    def _release(self):
        self._x = self._saved = None
