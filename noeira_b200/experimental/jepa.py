"""A joint-embedding predictive world model trained end to end from observations and actions, with no reconstruction, no
target network and no stop-gradient: an encoder maps observations to latents, an action-conditioned predictor maps
(latent, action) to the next latent, and the loss is the prediction error in latent space (gradient through BOTH sides)
plus a regulariser that keeps the batch of latents distributed like an isotropic Gaussian, which is what prevents the
collapse that the prediction term alone invites.

The regulariser (``sigreg``) sketches the distribution: project the latents on random unit directions, and for each
projection compare the empirical characteristic function with that of N(0, 1) at a few knots under a Gaussian window (the
Epps–Pulley statistic, by trapezoid rule).  A fresh set of directions is drawn every step.

Encoder and predictor are ``nn`` modules (their GEMMs are the tcgen05 kernels on CUDA); the loss graph runs under torch
autograd through ``nn.apply``, which hands the modules' own ``vjp`` to autograd and leaves parameter gradients in the
optimizer's arena.  ``plan`` is random-shooting model-predictive control toward a goal observation in latent space.

Reference: noeira/experimental/lewm/ (ref_model.mojo, ref_trainer.mojo: prediction loss + 0.09 × SIGReg with 1024
projections × 17 knots, BatchNorm projector, copy-last baseline of ``window_losses``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .. import nn


def sigreg(z: torch.Tensor, directions: torch.Tensor, knots: int = 17, t_max: float = 3.0) -> torch.Tensor:
    """Epps–Pulley distance between the projections of z [B, D] on ``directions`` [D, P] (unit columns) and N(0, 1):
    B · ∫ |φ_emp(t) − e^{−t²/2}|² e^{−t²/2} dt, averaged over the projections."""
    t = torch.linspace(-t_max, t_max, knots, device=z.device, dtype=z.dtype)
    p = z @ directions                                           # [B, P]
    arg = p[:, :, None] * t                                      # [B, P, K]
    re, im = torch.cos(arg).mean(0), torch.sin(arg).mean(0)      # [P, K]
    target = torch.exp(-0.5 * t * t)
    err = (re - target) ** 2 + im ** 2
    w = target.clone()
    w[0] *= 0.5
    w[-1] *= 0.5
    return z.shape[0] * (err * w).sum(1).mean() * float(t[1] - t[0])


def random_directions(d: int, p: int, gen: torch.Generator, device) -> torch.Tensor:
    a = torch.randn(d, p, generator=gen, device=device)
    return a / a.norm(dim=0, keepdim=True)


@dataclass
class JEPAConfig:
    obs_dim: int = 16
    act_dim: int = 2
    latent_dim: int = 16
    hidden: int = 128
    sigreg_lambda: float = 0.09
    projections: int = 256
    knots: int = 17
    lr: float = 1e-3
    seed: int = 0


class JEPAWorldModel:
    def __init__(self, cfg: JEPAConfig, device="cpu"):
        self.cfg, self.device = cfg, torch.device(device)
        torch.manual_seed(cfg.seed)
        c = cfg
        self.encoder = nn.Sequential(nn.Linear(c.obs_dim, c.hidden, act="gelu"), nn.Linear(c.hidden, c.hidden, act="gelu"),
                                     nn.Linear(c.hidden, c.latent_dim)).to(self.device)
        self.predictor = nn.Sequential(nn.Linear(c.latent_dim + c.act_dim, c.hidden, act="gelu"),
                                       nn.Linear(c.hidden, c.hidden, act="gelu"), nn.Linear(c.hidden, c.latent_dim)).to(self.device)
        self.net = nn.Sequential(self.encoder, self.predictor)     # one parameter walk for the optimizer and checkpoints
        self.opt = nn.AdamW(list(self.net.named_params()), lr=c.lr, device=self.device)
        self.gen = torch.Generator(device=self.device).manual_seed(c.seed)

    def encode(self, obs: torch.Tensor) -> torch.Tensor:
        with torch.no_grad():
            return self.encoder.forward(obs.to(self.device)).float()

    def predict(self, z: torch.Tensor, act: torch.Tensor) -> torch.Tensor:
        with torch.no_grad():
            return self.predictor.forward(torch.cat([z, act.to(self.device)], 1)).float()

    def losses(self, obs, act, next_obs, grad: bool = False):
        """→ (total, prediction, regulariser, copy-last baseline).  With ``grad`` the graph is kept for ``backward``."""
        B = obs.shape[0]
        both = torch.cat([obs, next_obs], 0).to(self.device)
        with torch.set_grad_enabled(grad):
            z = (nn.apply(self.encoder, both) if grad else self.encoder.forward(both)).float()
            zt, zn = z[:B], z[B:]
            inp = torch.cat([zt, act.to(self.device)], 1)
            pred = (nn.apply(self.predictor, inp) if grad else self.predictor.forward(inp)).float()
            pl = (pred - zn).pow(2).sum(1).mean()
            dirs = random_directions(self.cfg.latent_dim, self.cfg.projections, self.gen, self.device)
            sg = sigreg(z, dirs, self.cfg.knots)
            copy_last = (zt - zn).pow(2).sum(1).mean()
        return pl + self.cfg.sigreg_lambda * sg, pl, sg, copy_last

    def train_step(self, obs, act, next_obs) -> dict:
        self.opt.zero_grad()
        total, pl, sg, cl = self.losses(obs, act, next_obs, grad=True)
        total.backward()
        self.opt.step()
        return {"loss": float(total.detach()), "pred": float(pl.detach()), "sigreg": float(sg.detach()), "copy_last": float(cl.detach())}

    def rollout(self, obs: torch.Tensor, actions: torch.Tensor) -> torch.Tensor:
        """Latents after each of the actions [B, H, A] applied from ``obs`` [B, obs_dim] → [B, H, D]."""
        z, out = self.encode(obs), []
        for h in range(actions.shape[1]):
            z = self.predict(z, actions[:, h])
            out.append(z)
        return torch.stack(out, 1)

    def plan(self, obs: torch.Tensor, goal_obs: torch.Tensor, horizon: int = 8, samples: int = 256, act_scale: float = 1.0) -> torch.Tensor:
        """Random shooting: the first action of the sampled sequence whose final latent is closest to the goal's."""
        a = (torch.rand(samples, horizon, self.cfg.act_dim, generator=self.gen, device=self.device) * 2 - 1) * act_scale
        zf = self.rollout(obs.to(self.device).expand(samples, -1), a)[:, -1]
        best = (zf - self.encode(goal_obs.reshape(1, -1))).pow(2).sum(1).argmin()
        return a[best, 0]
