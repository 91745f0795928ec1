"""Predictive coding networks in the canonical (Bogacz) form.

Every layer holds a value node x_l; the layer below predicts it, μ_{l+1} = W_l f(x_l) + b_l, and the mismatch
ε_{l+1} = x_{l+1} − μ_{l+1} is the only signal that travels.  With the input clamped to x_0 and, in training, the output
clamped to the target, INFERENCE relaxes the hidden value nodes down the energy F = ½ Σ ‖ε_l‖²,

    dx_l = −ε_l + f′(x_l) ⊙ (W_lᵀ ε_{l+1}),

and LEARNING is local: the gradient of F for W_l at the relaxed state is −ε_{l+1} f(x_l)ᵀ, an outer product of quantities that
sit at the two ends of that connection.  The output error may carry a precision λ (F counts ½ λ ‖ε_L‖²): the relaxation is
linear in the errors, so making the target close to the prediction changes nothing, but a WEAK output clamp does: as λ → 0
the hidden value nodes stay at their feed-forward values and the local gradients divided by λ are the back-propagation
gradients (at λ = 1 they are a different descent direction and shorter, the hidden layers having absorbed part of the
error).

``PCBlock`` is one connection, ``PCSequential`` the stack, ``PCTrainer`` runs the phases (predict and errors, value update,
weight gradients into ``Param.grad``, step of an ``nn`` arena optimizer); ``spectral_norm_clamp`` and ``clip_grad_norm`` are
the stabilisers.  Tensor arithmetic throughout: runs on CPU or CUDA tensors alike.

Reference: noeira/experimental/pcn/ (predictive_model.mojo, pc_block.mojo, pc_sequential.mojo, pc_trainer.mojo,
pc_utils.mojo).
"""
from __future__ import annotations

import math
from typing import Iterator, List, Sequence, Tuple

import torch

from ..nn.param import Param

ACTIVATIONS = {
    "identity": (lambda x: x, lambda x: torch.ones_like(x)),
    "relu": (torch.relu, lambda x: (x > 0).to(x.dtype)),
    "tanh": (torch.tanh, lambda x: 1 - torch.tanh(x) ** 2),
    "swish": (lambda x: x * torch.sigmoid(x), lambda x: torch.sigmoid(x) * (1 + x * (1 - torch.sigmoid(x)))),
}


class PCBlock:
    """μ_next = W f(x) + b for one pair of adjacent layers."""

    def __init__(self, n_in: int, n_out: int, act: str = "tanh", device="cpu", seed: int = 0):
        self.n_in, self.n_out, self.act = n_in, n_out, act
        self.f, self.df = ACTIVATIONS[act]
        self.w = Param("w", (n_out, n_in), device=device, pad_rows=False)
        self.b = Param("b", (n_out,), decay=False, device=device, pad_rows=False)
        g = torch.Generator().manual_seed(seed)
        self.w.data.copy_(torch.randn(n_out, n_in, generator=g) * math.sqrt(1.0 / n_in))

    def predict(self, x: torch.Tensor) -> torch.Tensor:
        return self.f(x) @ self.w.data.T + self.b.data

    def back_error(self, x: torch.Tensor, eps_next: torch.Tensor) -> torch.Tensor:
        """f′(x) ⊙ (Wᵀ ε_next): what the error above asks of this layer's value node."""
        return self.df(x) * (eps_next @ self.w.data)

    def accumulate_grads(self, x: torch.Tensor, eps_next: torch.Tensor):
        """∂F/∂W = −ε_next f(x)ᵀ, ∂F/∂b = −ε_next, averaged over the batch."""
        n = x.shape[0]
        self.w.grad.add_(-(eps_next.T @ self.f(x)) / n)
        self.b.grad.add_(-eps_next.sum(0) / n)


class PCSequential:
    def __init__(self, sizes: Sequence[int], act: str = "tanh", first_act: str = "identity", device="cpu", seed: int = 0):
        """``sizes`` = widths of x_0 … x_L.  The input layer is passed through ``first_act`` (identity: data are not squashed)."""
        self.sizes = list(sizes)
        self.blocks: List[PCBlock] = [PCBlock(a, b, first_act if i == 0 else act, device, seed + i)
                                      for i, (a, b) in enumerate(zip(sizes[:-1], sizes[1:]))]

    def named_params(self) -> Iterator[Tuple[str, Param]]:
        for i, blk in enumerate(self.blocks):
            yield f"{i}.w", blk.w
            yield f"{i}.b", blk.b

    def forward(self, x0: torch.Tensor) -> List[torch.Tensor]:
        """The feed-forward pass: every value node at its prediction (all errors zero)."""
        xs = [x0]
        for blk in self.blocks:
            xs.append(blk.predict(xs[-1]))
        return xs

    def errors(self, xs: List[torch.Tensor]) -> List[torch.Tensor]:
        """ε_1 … ε_L"""
        return [xs[l + 1] - blk.predict(xs[l]) for l, blk in enumerate(self.blocks)]

    def energy(self, xs: List[torch.Tensor], output_precision: float = 1.0) -> torch.Tensor:
        eps = self.errors(xs)
        eps[-1] = eps[-1] * math.sqrt(output_precision)
        return 0.5 * sum(e.pow(2).sum(1) for e in eps).mean()


class PCTrainer:
    def __init__(self, net: PCSequential, lr: float = 1e-3, infer_steps: int = 20, infer_lr: float = 0.1, max_grad_norm: float = 0.0,
                 max_spectral_norm: float = 0.0, output_precision: float = 1.0):
        from ..nn.optim import Adam
        self.net, self.infer_steps, self.infer_lr = net, infer_steps, infer_lr
        self.max_grad_norm, self.max_spectral_norm, self.output_precision = max_grad_norm, max_spectral_norm, output_precision
        dev = net.blocks[0].w.data.device
        self.opt = Adam(list(net.named_params()), lr=lr, device=dev)

    def predict(self, x0: torch.Tensor) -> torch.Tensor:
        return self.net.forward(x0)[-1]

    def readout_loss(self, x0: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        return 0.5 * (self.predict(x0) - y).pow(2).sum(1).mean()

    def inference_step(self, xs: List[torch.Tensor], clamp_output: bool) -> List[torch.Tensor]:
        """One relaxation step of the free value nodes (x_0 is always clamped, x_L when ``clamp_output``)."""
        net = self.net
        eps = net.errors(xs)
        eps[-1] = eps[-1] * self.output_precision
        out = list(xs)
        last = len(xs) - 1
        for l in range(1, len(xs)):
            if l == last and clamp_output:
                continue
            dx = -eps[l - 1]
            if l < last:
                dx = dx + net.blocks[l].back_error(xs[l], eps[l])
            out[l] = xs[l] + self.infer_lr * dx
        return out

    def infer(self, x0: torch.Tensor, y: torch.Tensor = None, steps: int = None, trace: list = None) -> List[torch.Tensor]:
        xs = self.net.forward(x0)
        if y is not None:
            xs[-1] = y
        for _ in range(self.infer_steps if steps is None else steps):
            if trace is not None:
                trace.append(float(self.net.energy(xs, self.output_precision)))
            xs = self.inference_step(xs, clamp_output=y is not None)
        if trace is not None:
            trace.append(float(self.net.energy(xs, self.output_precision)))
        return xs

    def local_grads(self, xs: List[torch.Tensor]):
        eps = self.net.errors(xs)
        eps[-1] = eps[-1] * self.output_precision
        for l, blk in enumerate(self.net.blocks):
            blk.accumulate_grads(xs[l], eps[l])

    def train_step(self, x0: torch.Tensor, y: torch.Tensor) -> float:
        """Relax with input and target clamped, take the local gradients, step; returns the energy at the relaxed state."""
        xs = self.infer(x0, y)
        self.opt.zero_grad()
        self.local_grads(xs)
        if self.max_grad_norm > 0:
            clip_grad_norm([p for _, p in self.net.named_params()], self.max_grad_norm)
        self.opt.step()
        if self.max_spectral_norm > 0:
            for blk in self.net.blocks:
                spectral_norm_clamp(blk.w.data, self.max_spectral_norm)
        return float(self.net.energy(xs, self.output_precision))


def clip_grad_norm(params: Sequence[Param], max_norm: float) -> float:
    total = math.sqrt(sum(float(p.grad.pow(2).sum()) for p in params))
    if total > max_norm:
        for p in params:
            p.grad.mul_(max_norm / total)
    return total


def spectral_norm_clamp(w: torch.Tensor, max_norm: float, iters: int = 30) -> float:
    """Scale ``w`` in place so that its largest singular value (power iteration) is at most ``max_norm``; returns the value
    found before scaling."""
    v = torch.ones(w.shape[1], device=w.device, dtype=w.dtype) / math.sqrt(w.shape[1])
    sigma = 0.0
    for _ in range(iters):
        u = w @ v
        sigma = float(u.norm())
        if sigma == 0.0:
            return 0.0
        v = w.T @ (u / sigma)
        v = v / v.norm().clamp_min(1e-30)
    sigma = float((w @ v).norm())
    if sigma > max_norm:
        w.mul_(max_norm / sigma)
    return sigma
