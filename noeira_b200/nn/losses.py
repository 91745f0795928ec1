"""Losses with explicit gradients (tensor programs; the hot ones — MSE / L1, cross-entropy, KL — have CUDA kernels in
``nn.transformer``).  Each returns ``(loss scalar tensor, gradient w.r.t. the prediction)``.
Reference: noeira/nn/loss/ (GaussianNLLLoss, BCE, two_hot.mojo symlog two-hot targets, per-sample reductions)."""
from __future__ import annotations

import math

import torch


def gaussian_nll(mean, log_std, target, min_log_std=-10.0, max_log_std=2.0):
    """Mean over elements of 0.5·((t−μ)/σ)² + log σ + 0.5·log 2π.  → (loss, dmean, dlog_std)"""
    ls = log_std.float().clamp(min_log_std, max_log_std)
    inv = torch.exp(-ls)
    z = (target.float() - mean.float()) * inv
    n = z.numel()
    loss = (0.5 * z * z + ls + 0.5 * math.log(2 * math.pi)).mean()
    inside = ((log_std.float() >= min_log_std) & (log_std.float() <= max_log_std)).float()
    return loss, (-z * inv) / n, ((1 - z * z) * inside) / n


def bce_with_logits(logits, target):
    x, t = logits.float(), target.float()
    loss = (torch.clamp(x, min=0) - x * t + torch.log1p(torch.exp(-x.abs()))).mean()
    return loss, (torch.sigmoid(x) - t) / x.numel()


def symlog(x):
    return torch.sign(x) * torch.log1p(x.abs())


def symexp(x):
    return torch.sign(x) * torch.expm1(x.abs())


def two_hot(target, bins: torch.Tensor):
    """Scalar targets → probability over ``bins`` (ascending) with mass on the two neighbouring bins."""
    t = target.float().clamp(bins[0], bins[-1])
    hi = torch.searchsorted(bins, t.contiguous(), right=True).clamp(1, len(bins) - 1)
    lo = hi - 1
    w_hi = (t - bins[lo]) / (bins[hi] - bins[lo])
    out = torch.zeros(*t.shape, len(bins), device=t.device)
    out.scatter_(-1, lo.unsqueeze(-1), (1 - w_hi).unsqueeze(-1))
    out.scatter_add_(-1, hi.unsqueeze(-1), w_hi.unsqueeze(-1))
    return out


def two_hot_loss(logits, target, bins: torch.Tensor, use_symlog: bool = True):
    """Cross-entropy between softmax(logits) and the two-hot encoding of (symlog) targets. → (loss, dlogits)"""
    t = symlog(target.float()) if use_symlog else target.float()
    p = two_hot(t, bins)
    logp = torch.log_softmax(logits.float(), -1)
    n = max(t.numel(), 1)
    return -(p * logp).sum(-1).mean(), (torch.softmax(logits.float(), -1) - p) / n


def two_hot_decode(logits, bins: torch.Tensor, use_symlog: bool = True):
    v = (torch.softmax(logits.float(), -1) * bins).sum(-1)
    return symexp(v) if use_symlog else v


def mse_per_sample(pred, target):
    d = pred.float() - target.float()
    per = d.reshape(d.shape[0], -1).pow(2).mean(1)
    return per, 2 * d / d[0].numel()


def l1_masked_per_sample(pred, target, mask):
    """``mask [B, T]`` selects valid steps; mean over valid elements of each sample."""
    d = (pred.float() - target.float()) * mask.float().unsqueeze(-1)
    cnt = (mask.float().sum(1) * pred.shape[-1]).clamp_min(1.0)
    per = d.abs().reshape(d.shape[0], -1).sum(1) / cnt
    return per, torch.sign(d) / cnt.reshape(-1, *([1] * (d.dim() - 1)))
