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
        """Update k of the K updates that follow one collection phase samples from the most recent c_k = max(N·eta^(k·1000/K), c_min) items."""
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


class StoreReplayGpu:
    """Device ring of packed transitions ``[s | a | r | s' | d]`` driven entirely by kernels (``csrc/replay.cu``): the write
    offset, the size and the sampling counter live in a device ``meta`` block, so ``store`` → ``sample`` → update can be
    captured in one CUDA graph.  Sampling: ``"uniform"``, ``"ere"`` (pass the fraction ``eta^(k·1000/K)``), ``"per"`` (sum
    tree; ``update_priorities`` after the TD errors are known).  (noeira/data/replay_gpu.mojo:54-330)"""

    def __init__(self, capacity: int, obs_dim: int, act_dim: int, demo_prefix: int = 0, seed: int = 0, per_alpha: float = 0.6,
                 per_beta: float = 0.4, device="cuda", prioritized: bool = True):
        import ctypes
        from .._native import cuda_lib
        self._c, self._lib = ctypes, cuda_lib()
        self.capacity, self.obs_dim, self.act_dim, self.base = capacity, obs_dim, act_dim, demo_prefix
        self.width = 2 * obs_dim + act_dim + 2
        self.device = torch.device(device)
        self.buf = torch.zeros(capacity, self.width, device=self.device)
        self.meta = torch.tensor([demo_prefix, demo_prefix, 0], dtype=torch.int64, device=self.device)
        self.seed, self.per_alpha, self.per_beta = seed, per_alpha, per_beta
        # the sum tree is maintained only when prioritized sampling is in use (uniform / ERE never read it)
        self.prioritized = prioritized and per_alpha > 0
        self.leaves = 1
        while self.leaves < capacity:
            self.leaves *= 2
        self.tree = torch.zeros(2 * self.leaves if self.prioritized else 2, device=self.device)
        self._idx, self._out, self._w = {}, {}, {}

    def _ptr(self, t):
        from .._native import ptr
        return ptr(t)

    def store_batch(self, s, a, r, sp, d):
        from .._native import check, stream_ptr
        rows = torch.cat([s.float(), a.float(), r.float().reshape(-1, 1), sp.float(), d.float().reshape(-1, 1)], 1).contiguous()
        c = self._c
        n = rows.shape[0]
        if self.prioritized:
            # new transitions enter with the running maximum priority: here priority 1 before the exponent
            start = self.meta[0:1].clone()
        check(self._lib.nb_replay_store(self._ptr(self.buf), c.c_int(self.width), c.c_longlong(self.capacity), self._ptr(self.meta),
                                        self._ptr(rows), c.c_int(n), c.c_int(self.base), stream_ptr()), "replay_store")
        if self.prioritized:
            ring = self.capacity - self.base
            idx = (start - self.base + torch.arange(n, device=self.device)) % ring + self.base
            self.update_priorities(idx, torch.ones(n, device=self.device))

    def indices(self, batch: int, mode: str = "uniform", ere_frac: float = 1.0, c_min: int = 5000):
        from .._native import check, stream_ptr
        c = self._c
        idx = self._idx.setdefault(batch, torch.zeros(batch, dtype=torch.int64, device=self.device))
        if mode == "per":
            assert self.prioritized, "construct the store with prioritized=True to sample by priority"
            w = self._w.setdefault(batch, torch.zeros(batch, device=self.device))
            check(self._lib.nb_per_sample(self._ptr(self.tree), c.c_longlong(self.leaves), self._ptr(idx), self._ptr(w),
                                          c.c_int(batch), self._ptr(self.meta), c.c_ulonglong(self.seed),
                                          c.c_float(self.per_beta), stream_ptr()), "per_sample")
            return idx, w / w.max()
        check(self._lib.nb_replay_indices(self._ptr(idx), c.c_int(batch), self._ptr(self.meta), c.c_ulonglong(self.seed),
                                          c.c_int(0 if mode == "uniform" else 1), c.c_float(ere_frac), c.c_longlong(c_min),
                                          c.c_longlong(self.capacity), c.c_int(self.base), stream_ptr()), "replay_indices")
        return idx, None

    def update_priorities(self, idx, td_abs):
        from .._native import check, stream_ptr
        c = self._c
        check(self._lib.nb_per_update(self._ptr(self.tree), c.c_longlong(self.leaves), self._ptr(idx.contiguous()),
                                      self._ptr(td_abs.float().contiguous()), c.c_int(idx.numel()), c.c_float(self.per_alpha),
                                      c.c_float(1e-6), stream_ptr()), "per_update")

    def gather(self, idx):
        from .._native import check, stream_ptr
        c = self._c
        b = idx.numel()
        out = self._out.setdefault(b, torch.zeros(b, self.width, device=self.device))
        check(self._lib.nb_replay_gather(self._ptr(self.buf), c.c_int(self.width), self._ptr(idx), self._ptr(out), c.c_int(b),
                                         c.c_longlong(self.capacity), stream_ptr()), "replay_gather")
        O, A = self.obs_dim, self.act_dim
        return out[:, :O], out[:, O:O + A], out[:, O + A], out[:, O + A + 1: 2 * O + A + 1], out[:, 2 * O + A + 1]

    def sample(self, batch: int, mode: str = "uniform", **kw):
        idx, w = self.indices(batch, mode, **kw)
        return self.gather(idx), idx, w

    @property
    def size(self) -> int:
        return int(self.meta[1])
