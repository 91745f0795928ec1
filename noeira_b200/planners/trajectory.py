"""Sampling-based trajectory optimisers over a batched rollout function.

A rollout function maps ``actions [K, H, A]`` to ``returns [K]`` (one candidate sequence per batch lane); the planners
only need that, so the same code plans on an analytic model, on the batched physics engine (``PhysicsRollout``:
K lanes of the engine are reset to the current state and stepped H times on the device) or on a learned world model.
``MPPI``: exponentially weighted update of the mean sequence with temperature λ, warm-started by shifting one step;
``CEM``: refit mean / std to the elites for a few iterations; ``RandomShooting``: best of K.
Reference: noeira/planners/trajectory/ (mppi.mojo + mppi_kernels.mojo GPU batched variant, cem.mojo, random_shooter.mojo).
"""
from __future__ import annotations

from typing import Callable

import torch


class _Planner:
    def __init__(self, rollout: Callable, horizon: int, act_dim: int, samples: int, act_low=-1.0, act_high=1.0,
                 device="cpu", seed: int = 0):
        self.rollout, self.H, self.A, self.K = rollout, horizon, act_dim, samples
        self.low, self.high = act_low, act_high
        self.device = torch.device(device)
        self.gen = torch.Generator(device=self.device).manual_seed(seed)
        self.mean = torch.zeros(horizon, act_dim, device=self.device)

    def _noise(self, *shape):
        return torch.randn(*shape, device=self.device, generator=self.gen)

    def shift(self):
        """Warm start for the next control step: drop the executed action, repeat the last one."""
        self.mean = torch.cat([self.mean[1:], self.mean[-1:]], 0)


class MPPI(_Planner):
    def __init__(self, rollout, horizon, act_dim, samples=256, sigma=0.5, lam=1.0, **kw):
        super().__init__(rollout, horizon, act_dim, samples, **kw)
        self.sigma, self.lam = sigma, lam

    def plan(self, iterations: int = 1) -> torch.Tensor:
        for _ in range(iterations):
            eps = self._noise(self.K, self.H, self.A) * self.sigma
            eps[0] = 0                                           # lane 0 evaluates the current mean itself
            acts = (self.mean[None] + eps).clamp(self.low, self.high)
            ret = self.rollout(acts).float()
            w = torch.softmax((ret - ret.max()) / self.lam, 0)
            self.mean = (w[:, None, None] * acts).sum(0)
        return self.mean[0].clone()


class CEM(_Planner):
    def __init__(self, rollout, horizon, act_dim, samples=256, elites=32, init_std=0.7, min_std=0.05, momentum=0.1, **kw):
        super().__init__(rollout, horizon, act_dim, samples, **kw)
        self.n_elite, self.init_std, self.min_std, self.momentum = elites, init_std, min_std, momentum

    def plan(self, iterations: int = 4) -> torch.Tensor:
        std = torch.full_like(self.mean, self.init_std)
        for _ in range(iterations):
            acts = (self.mean[None] + self._noise(self.K, self.H, self.A) * std[None]).clamp(self.low, self.high)
            ret = self.rollout(acts).float()
            elite = acts[ret.topk(self.n_elite).indices]
            self.mean = self.momentum * self.mean + (1 - self.momentum) * elite.mean(0)
            std = elite.std(0).clamp_min(self.min_std)
        return self.mean[0].clone()


class RandomShooting(_Planner):
    def plan(self, iterations: int = 1) -> torch.Tensor:
        acts = torch.rand(self.K, self.H, self.A, device=self.device, generator=self.gen) * (self.high - self.low) + self.low
        ret = self.rollout(acts).float()
        self.mean = acts[ret.argmax()]
        return self.mean[0].clone()


class PhysicsRollout:
    """Rollout function over the lanes of a batched physics environment: every lane starts from ``(qpos, qvel)`` of the
    controlled system, lane k applies ``actions[k]`` for H steps, the discounted reward sum comes back; episode resets are
    off during planning rollouts (termination only ends that lane's accumulation)."""

    def __init__(self, env, gamma: float = 0.99):
        self.env, self.gamma = env, gamma
        self.state = None

    def set_state(self, qpos: torch.Tensor, qvel: torch.Tensor):
        self.state = (qpos.clone(), qvel.clone())

    def __call__(self, actions: torch.Tensor) -> torch.Tensor:
        env = self.env
        K, H, _ = actions.shape
        assert K == env.n_envs
        e = env.engine
        e.qpos.copy_(self.state[0].expand_as(e.qpos))
        e.qvel.copy_(self.state[1].expand_as(e.qvel))
        e.warm.zero_()
        e.step_count.zero_()
        total = torch.zeros(K, device=actions.device)
        alive = torch.ones(K, device=actions.device)
        disc = 1.0
        for t in range(H):
            env.step_batch(actions[:, t].contiguous(), auto_reset=False)
            total += disc * alive * env.reward
            alive = alive * (1.0 - env.terminated)
            disc *= self.gamma
        return total
