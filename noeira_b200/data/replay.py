"""Replay buffers: a ring of transitions resident on the training device (CPU or GPU).

``StoreReplay`` keeps ``s, a, r, s', done`` as preallocated tensors; ``store_batch`` writes N_ENVS transitions
to consecutive slots with wrap-around inside ``[base, capacity)`` where ``base`` is an optional pinned demo
prefix; sampling policies: uniform, ERE (emphasising recent experience) and PER (proportional, sum-tree free:
prefix-sum sampling over priorities with importance weights normalised by their maximum).
Reference: noeira/data/replay.mojo:39 (CPU), noeira/data/replay_gpu.mojo:82-482 (device ring, uniform / ERE /
PER index kernels, mixed demo/online draws).
"""
from __future__ import annotations

import torch


class StoreReplay:
    def __init__(self, capacity: int, obs_dim: int, act_dim: int, device="cpu", demo_prefix: int = 0, seed: int = 0,
                 per_alpha: float = 0.6, per_beta: float = 0.4):
        self.capacity, self.obs_dim, self.act_dim = capacity, obs_dim, act_dim
        self.device = torch.device(device)
        z = dict(device=self.device, dtype=torch.float32)
        self.s = torch.zeros(capacity, obs_dim, **z)
        self.sp = torch.zeros(capacity, obs_dim, **z)
        self.a = torch.zeros(capacity, act_dim, **z)
        self.r = torch.zeros(capacity, **z)
        self.d = torch.zeros(capacity, **z)
        self.prio = torch.zeros(capacity, **z)
        self.base = demo_prefix
        self.pos = demo_prefix
        self.size = demo_prefix
        self.max_prio = 1.0
        self.per_alpha, self.per_beta = per_alpha, per_beta
        self.gen = torch.Generator(device=self.device).manual_seed(seed)

    def store_batch(self, s, a, r, sp, d):
        n = s.shape[0]
        idx = (torch.arange(n, device=self.device) + (self.pos - self.base)) % (self.capacity - self.base) + self.base
        self.s[idx], self.a[idx], self.r[idx], self.sp[idx], self.d[idx] = s, a, r, sp, d
        self.prio[idx] = self.max_prio
        self.pos = int((self.pos - self.base + n) % (self.capacity - self.base) + self.base)
        self.size = min(self.capacity, self.size + n)
        return idx

    def uniform_indices(self, batch):
        return torch.randint(0, max(self.size, 1), (batch,), device=self.device, generator=self.gen)

    def ere_indices(self, batch, k, K, eta=0.996, c_min=5000):
        """Update k of K in this round samples from the most recent c_k = max(N·eta^(k·1000/K), c_min) items."""
        ck = int(max(self.size * eta ** (k * 1000.0 / max(K, 1)), min(c_min, self.size)))
        off = torch.randint(0, max(ck, 1), (batch,), device=self.device, generator=self.gen)
        return (self.pos - 1 - off) % max(self.size, 1)

    def per_indices(self, batch):
        p = self.prio[: self.size].clamp_min(1e-8) ** self.per_alpha
        cdf = torch.cumsum(p, 0)
        u = torch.rand(batch, device=self.device, generator=self.gen) * cdf[-1]
        idx = torch.searchsorted(cdf, u).clamp_max(self.size - 1)
        w = (self.size * p[idx] / cdf[-1]) ** (-self.per_beta)
        return idx, w / w.max()

    def update_priorities(self, idx, td_abs):
        self.prio[idx] = td_abs.abs() + 1e-6
        self.max_prio = max(self.max_prio, float(self.prio[idx].max()))

    def mixed_indices(self, batch, demo_fraction=0.5):
        """Half demo prefix / half online draws (HIL-SERL / RLPD style)."""
        nd = int(batch * demo_fraction) if self.base > 0 else 0
        di = torch.randint(0, max(self.base, 1), (nd,), device=self.device, generator=self.gen)
        oi = torch.randint(self.base, max(self.size, self.base + 1), (batch - nd,), device=self.device, generator=self.gen)
        return torch.cat([di, oi])

    def gather(self, idx):
        return self.s[idx], self.a[idx], self.r[idx], self.sp[idx], self.d[idx]

    def sample(self, batch):
        return self.gather(self.uniform_indices(batch))
