"""Initializers (reference: noeira/nn/core/initializer.mojo:32-232).  Each is a callable
``init(shape, fan_in, fan_out, generator) -> fp32 tensor`` evaluated on the CPU for determinism."""
from __future__ import annotations

import math

import torch


class Initializer:
    def __call__(self, shape, fan_in, fan_out, gen):
        raise NotImplementedError


class Kaiming(Initializer):
    """U(-1/sqrt(fan_in), 1/sqrt(fan_in)) — the torch.nn.Linear default."""

    def __call__(self, shape, fan_in, fan_out, gen):
        b = 1.0 / math.sqrt(max(fan_in, 1))
        return (torch.rand(shape, generator=gen) * 2 - 1) * b


class ScaledKaiming(Initializer):
    def __init__(self, scale: float):
        self.scale = scale

    def __call__(self, shape, fan_in, fan_out, gen):
        return Kaiming()(shape, fan_in, fan_out, gen) * self.scale


class Xavier(Initializer):
    def __call__(self, shape, fan_in, fan_out, gen):
        b = math.sqrt(6.0 / max(fan_in + fan_out, 1))
        return (torch.rand(shape, generator=gen) * 2 - 1) * b


class TruncNormalIn(Initializer):
    """N(0, 1/fan_in) truncated at 2 sigma."""

    def __call__(self, shape, fan_in, fan_out, gen):
        std = 1.0 / math.sqrt(max(fan_in, 1))
        t = torch.empty(shape)
        torch.nn.init.trunc_normal_(t, 0.0, std, -2 * std, 2 * std, generator=gen)
        return t


class Normal(Initializer):
    def __init__(self, mean=0.0, std=0.02):
        self.mean, self.std = mean, std

    def __call__(self, shape, fan_in, fan_out, gen):
        return torch.randn(shape, generator=gen) * self.std + self.mean


class Zero(Initializer):
    def __call__(self, shape, fan_in, fan_out, gen):
        return torch.zeros(shape)


class Constant(Initializer):
    def __init__(self, v):
        self.v = v

    def __call__(self, shape, fan_in, fan_out, gen):
        return torch.full(shape, float(self.v))


class Deterministic(Initializer):
    """sin-pattern used by bit-exact parity gates (no RNG)."""

    def __call__(self, shape, fan_in, fan_out, gen):
        n = 1
        for s in shape:
            n *= s
        i = torch.arange(n, dtype=torch.float32)
        return (torch.sin(i * 0.37 + 0.11) * 0.5 / math.sqrt(max(fan_in, 1))).reshape(shape)


class Orthogonal(Initializer):
    def __init__(self, gain=1.0):
        self.gain = gain

    def __call__(self, shape, fan_in, fan_out, gen):
        t = torch.empty(shape)
        torch.nn.init.orthogonal_(t, gain=self.gain, generator=gen)
        return t
