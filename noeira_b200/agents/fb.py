"""Forward-backward representations: reward-free pre-training of a family of policies, zero-shot transfer to any reward.

Networks (``nn`` modules applied through ``nn.apply``): two forward maps ``F_i(s, a, z) ∈ R^d``, a backward map
``B(s) ∈ R^d`` (rows L2-normalised to radius √d), an actor ``π(s, z)``.  For task vectors z drawn on the sphere of radius
√d (half of them from ``B`` of batch states), ``F(s, a, z)ᵀ B(s')`` is trained to be the successor measure of π_z:

  L_FB = ½ E_{s, s⁺}[(F(s, a, z)ᵀ B(s⁺) − γ F̄(s', π(s', z), z)ᵀ B̄(s⁺))²]_{off-diagonal} − E[F(s, a, z)ᵀ B(s')]
  L_ortho = E_{s≠s⁺}[(B(s)ᵀ B(s⁺))²] − 2 E[B(s)ᵀ B(s)]                       (keeps B's covariance near identity)
  L_actor = − E[min_i F_i(s, π(s, z), z)ᵀ z]

Targets F̄, B̄ follow by Polyak averaging.  At test time a reward function is turned into a task vector without any further
learning: ``z_r = E_s[r(s) B(s)]`` rescaled to the sphere, and the agent acts with π(·, z_r); the predicted value is
``F(s, a, z_r)ᵀ z_r``.   (noeira/deep_agents/fb/.)
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict

import torch

from .. import nn


@dataclass
class FBConfig:
    obs_dim: int = 3
    act_dim: int = 1
    z_dim: int = 16
    hidden: int = 128
    batch: int = 128
    lr: float = 3e-4
    gamma: float = 0.98
    tau: float = 0.01
    ortho_coef: float = 1.0
    mix_ratio: float = 0.5            # share of task vectors taken from B(states) instead of the uniform sphere
    actor_std: float = 0.2
    max_grad_norm: float = 10.0
    seed: int = 0


def _mlp(i, h, o, need_in=True):
    return nn.Sequential(nn.Linear(i, h, act="relu", need_input_grad=need_in), nn.Linear(h, h, act="relu"), nn.Linear(h, o, out_fp32=True))


def _project(z, d):
    return math.sqrt(d) * torch.nn.functional.normalize(z, dim=-1)


class FBAgent:
    def __init__(self, cfg: FBConfig = None, device="cpu"):
        self.cfg = c = cfg or FBConfig()
        self.device = torch.device(device)
        nn.manual_seed(c.seed)
        O, A, Z, H = c.obs_dim, c.act_dim, c.z_dim, c.hidden
        mk_f = lambda: _mlp(O + A + Z, H, Z).to(self.device)
        self.f1, self.f2, self.f1t, self.f2t = mk_f(), mk_f(), mk_f(), mk_f()
        self.b, self.bt = _mlp(O, H, Z, need_in=False).to(self.device), _mlp(O, H, Z, need_in=False).to(self.device)
        self.actor = _mlp(O + Z, H, A).to(self.device)
        for t, o in ((self.f1t, self.f1), (self.f2t, self.f2), (self.bt, self.b)):
            t.copy_from(o)
        self.fb_opt = nn.Adam(list(self.f1.named_params("f1.")) + list(self.f2.named_params("f2.")) + list(self.b.named_params("b.")), lr=c.lr)
        self.actor_opt = nn.Adam(self.actor.named_params("actor."), lr=c.lr)
        self.fb_opt.max_grad_norm = self.actor_opt.max_grad_norm = c.max_grad_norm
        self.gen = torch.Generator(device=self.device).manual_seed(c.seed + 1)
        self.last: Dict[str, float] = {}

    def _x(self, t):
        return t.to(torch.bfloat16) if self.device.type == "cuda" else t.float()

    # ------------------------------------------------------------------ pieces
    def backward_map(self, net, s, call):
        return _project(call(net, self._x(s)).float(), self.cfg.z_dim)

    def forward_map(self, net, s, a, z, call):
        return call(net, self._x(torch.cat([s, a, z], -1))).float()

    def policy(self, s, z, call, noise=True):
        mu = torch.tanh(call(self.actor, self._x(torch.cat([s, z], -1))).float())
        if not noise:
            return mu
        eps = torch.randn(mu.shape, device=self.device, generator=self.gen) * self.cfg.actor_std
        return (mu + eps.clamp(-0.3, 0.3)).clamp(-1, 1)

    @staticmethod
    def _fwd(module, *xs):
        return module.forward(*xs)

    def sample_z(self, n, states=None):
        c = self.cfg
        z = _project(torch.randn(n, c.z_dim, device=self.device, generator=self.gen), c.z_dim)
        if states is not None and c.mix_ratio > 0:
            with torch.no_grad():
                zb = self.backward_map(self.b, states[torch.randperm(states.shape[0], device=self.device, generator=self.gen)[:n]], self._fwd)
            pick = torch.rand(n, device=self.device, generator=self.gen) < c.mix_ratio
            z = torch.where(pick[:, None], zb, z)
        return z

    # ------------------------------------------------------------------ zero-shot inference
    @torch.no_grad()
    def infer_z(self, states, rewards):
        """Task vector of a reward function from labelled states: z = normalise(E[r(s) B(s)])."""
        B = self.backward_map(self.b, states.to(self.device).float(), self._fwd)
        return _project((rewards.to(self.device).float()[:, None] * B).mean(0, keepdim=True), self.cfg.z_dim)[0]

    @torch.no_grad()
    def select_action(self, obs, z, explore=False):
        s = obs.to(self.device).float()
        return self.policy(s, z.expand(s.shape[0], -1), self._fwd, noise=explore)

    @torch.no_grad()
    def value(self, s, a, z):
        zz = z.expand(s.shape[0], -1)
        return torch.minimum((self.forward_map(self.f1, s, a, zz, self._fwd) * zz).sum(-1), (self.forward_map(self.f2, s, a, zz, self._fwd) * zz).sum(-1))

    # ------------------------------------------------------------------ training
    def update(self, s, a, sp, d=None):
        """One reward-free update from transitions ``(s, a, s')`` (``d``: terminal flags)."""
        c, n = self.cfg, s.shape[0]
        s, a, sp = s.float(), a.float(), sp.float()
        disc = c.gamma * (1 - d.float()) if d is not None else torch.full((n,), c.gamma, device=self.device)
        z = self.sample_z(n, sp)
        eye = torch.eye(n, device=self.device, dtype=torch.bool)
        with torch.no_grad():
            ap = self.policy(sp, z, self._fwd)
            Bt = self.backward_map(self.bt, sp, self._fwd)                                    # [n, d]
            Mt = torch.minimum(self.forward_map(self.f1t, sp, ap, z, self._fwd) @ Bt.T, self.forward_map(self.f2t, sp, ap, z, self._fwd) @ Bt.T)
        Bn = self.backward_map(self.b, sp, nn.apply)
        fb_loss = 0.0
        for f in (self.f1, self.f2):
            M = self.forward_map(f, s, a, z, nn.apply) @ Bn.T                                  # M[i, j] = F(s_i, a_i, z_i)ᵀ B(s'_j)
            diff = M - disc[:, None] * Mt
            fb_loss = fb_loss + 0.5 * diff[~eye].pow(2).mean() - M.diagonal().mean()
        cov = Bn @ Bn.T
        ortho = cov[~eye].pow(2).mean() - 2 * cov.diagonal().mean()
        loss = fb_loss + c.ortho_coef * ortho
        loss.backward()
        if c.max_grad_norm > 0:
            self.fb_opt.clip()
        self.fb_opt.step(zero_grad=True)
        # ---- actor on detached states and task vectors
        ai = self.policy(s, z, nn.apply)
        q = torch.minimum((self.forward_map(self.f1, s, ai, z, nn.apply) * z).sum(-1), (self.forward_map(self.f2, s, ai, z, nn.apply) * z).sum(-1))
        aloss = -q.mean()
        aloss.backward()
        if c.max_grad_norm > 0:
            self.actor_opt.clip()
        self.actor_opt.step(zero_grad=True)
        self.fb_opt.arena.grd.zero_()                       # the forward maps only carried the gradient to the actor
        for t, o in ((self.f1t, self.f1), (self.f2t, self.f2), (self.bt, self.b)):
            t.polyak_from(o, c.tau)
        self.last = dict(fb_loss=float(fb_loss.detach()), ortho=float(ortho.detach()), actor_loss=float(aloss.detach()),
                         b_cov_offdiag=float(cov.detach()[~eye].abs().mean()))
        return self.last
