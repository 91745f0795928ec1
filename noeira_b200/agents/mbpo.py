"""MBPO: short model rollouts branched from real states feed a SAC learner.

``DynamicsEnsemble``  K probabilistic networks evaluated as ONE network of ``nn.BlockLinear`` layers (input
                      ``[B, K, obs+act]``): each member predicts mean and log-variance of ``[Δs, r]``; the log-variance is
                      soft-clamped between two learnable bounds; the loss is the Gaussian negative log-likelihood summed
                      over members plus a small pull on the bounds; every member sees its own bootstrap resample; inputs
                      are standardised by a scaler fitted on the training set; after training the ``elites`` members with
                      the lowest hold-out error are kept for rollouts.
``MBPOTrainer``       owns a ``SACTrainer``, the real replay and the model replay; ``train_model`` fits the ensemble,
                      ``rollout_model`` branches ``rollout_batch`` real states for ``rollout_len`` policy steps through a
                      random elite per sample and stores the imagined transitions, ``update`` draws ``real_ratio`` of each
                      batch from the real replay and the rest from the model replay.
``run_mbpo``          the collection / model-fit / rollout / update loop on a batched env.

(noeira/deep_agents/mbpo/: dynamics_ensemble_block.mojo — split / soft-clamp / learnable-bound NLL kernels;
trainer.mojo — posterior rollout, elite assignment and gather, scaler fit, target build.)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F

from .. import nn
from ..data.replay import StoreReplay
from .sac import SACConfig, SACTrainer


@dataclass
class MBPOConfig(SACConfig):
    ensemble: int = 7
    elites: int = 5
    model_hidden: int = 200
    model_layers: int = 3
    model_lr: float = 1e-3
    model_weight_decay: float = 1e-5
    model_batch: int = 256
    model_epochs: int = 5              # passes over the real replay per fit (the early-stopping criterion is the hold-out)
    holdout_fraction: float = 0.2
    bound_coef: float = 0.01
    model_train_every: int = 250       # env steps between two fits
    rollout_batch: int = 400
    rollout_len: int = 1
    real_ratio: float = 0.05
    model_retain: int = 100_000        # capacity of the model replay
    updates_per_step: int = 20


class DynamicsEnsemble(nn.Module):
    def __init__(self, obs_dim: int, act_dim: int, cfg: MBPOConfig):
        super().__init__()
        K, H = cfg.ensemble, cfg.model_hidden
        self.K, self.in_dim, self.out_dim = K, obs_dim + act_dim, obs_dim + 1
        layers, d = [], self.in_dim
        for i in range(cfg.model_layers):
            layers.append(nn.BlockLinear(d, H, K, act="silu", need_input_grad=i > 0))
            d = H
        layers.append(nn.BlockLinear(d, 2 * self.out_dim, K))
        self.net = self.add_child("net", nn.Sequential(*layers))
        self.max_logvar = self.add_param("max_logvar", (self.out_dim,), decay=False, init=nn.Constant(0.5))
        self.min_logvar = self.add_param("min_logvar", (self.out_dim,), decay=False, init=nn.Constant(-10.0))
        self.mu_in = torch.zeros(self.in_dim)
        self.sd_in = torch.ones(self.in_dim)
        self.elite_idx = torch.arange(min(cfg.elites, K))
        self.bound_coef = cfg.bound_coef

    def _moved(self, device):
        self.mu_in, self.sd_in, self.elite_idx = self.mu_in.to(device), self.sd_in.to(device), self.elite_idx.to(device)

    def fit_scaler(self, x):
        self.mu_in = x.mean(0)
        self.sd_in = x.std(0).clamp_min(1e-6)

    def forward(self, x):
        """x ``[B, K, in]`` (or ``[B, in]`` shared by all members) → mean, log-variance ``[B, K, out]``."""
        xs = (x.float() - self.mu_in) / self.sd_in
        raw = self.net.forward(xs).float()
        mean, r = raw[..., : self.out_dim], raw[..., self.out_dim:]
        mx, mn = self.max_logvar.data.float(), self.min_logvar.data.float()
        lv1 = mx - F.softplus(mx - r)
        lv = mn + F.softplus(lv1 - mn)
        self._cache = (r, lv1)
        return mean, lv

    def nll(self, mean, lv, y):
        """Σ_k mean_{b,d} [(μ − y)² e^{−lv} + lv] + c (Σ max − Σ min); returns the loss and its gradients w.r.t. mean / lv."""
        B, K, D = mean.shape
        inv = torch.exp(-lv)
        e2 = (mean - y) ** 2
        loss = (e2 * inv + lv).mean((0, 2)).sum() + self.bound_coef * (self.max_logvar.data.sum() - self.min_logvar.data.sum())
        return loss, 2 * (mean - y) * inv / (B * D), (1 - e2 * inv) / (B * D)

    def vjp(self, dmean, dlv):
        r, lv1 = self._cache
        mx, mn = self.max_logvar.data.float(), self.min_logvar.data.float()
        s2 = torch.sigmoid(lv1 - mn)                       # d lv / d lv1
        s1 = torch.sigmoid(mx - r)                         # d lv1 / d raw
        dlv1 = dlv * s2
        self.min_logvar.grad.add_((dlv * (1 - s2)).sum((0, 1)) - self.bound_coef)
        self.max_logvar.grad.add_((dlv1 * (1 - s1)).sum((0, 1)) + self.bound_coef)
        return self.net.vjp(torch.cat([dmean, dlv1 * s1], -1))

    @torch.no_grad()
    def predict(self, s, a, generator=None, deterministic=False):
        """One imagined step through a random elite per sample: ``(s', r)``."""
        B = s.shape[0]
        mean, lv = self.forward(torch.cat([s.float(), a.float()], 1))
        pick = self.elite_idx[torch.randint(0, self.elite_idx.numel(), (B,), device=s.device, generator=generator)]
        ar = torch.arange(B, device=s.device)
        m, sd = mean[ar, pick], torch.exp(0.5 * lv[ar, pick])
        out = m if deterministic else m + sd * torch.randn(m.shape, device=s.device, generator=generator)
        return s.float() + out[:, :-1], out[:, -1]


class MBPOTrainer:
    def __init__(self, cfg: MBPOConfig = None, device="cpu", capacity: int = 100_000,
                 termination_fn: Optional[Callable] = None):
        self.cfg = cfg = cfg or MBPOConfig()
        self.device = torch.device(device)
        self.sac = SACTrainer(cfg, device)
        nn.manual_seed(cfg.seed + 100)
        self.model = DynamicsEnsemble(cfg.obs_dim, cfg.act_dim, cfg).to(self.device)
        self.model_opt = nn.AdamW(self.model.named_params(), lr=cfg.model_lr, weight_decay=cfg.model_weight_decay)
        self.real = StoreReplay(capacity, cfg.obs_dim, cfg.act_dim, device=self.device, seed=cfg.seed)
        self.imagined = StoreReplay(cfg.model_retain, cfg.obs_dim, cfg.act_dim, device=self.device, seed=cfg.seed + 1)
        self.termination_fn = termination_fn or (lambda s, a, sp: torch.zeros(s.shape[0], device=s.device))
        self.gen = torch.Generator(device=self.device).manual_seed(cfg.seed + 2)
        self.holdout_mse = None
        self.metrics = {}

    # SAC surface
    def select_action(self, obs, deterministic=False):
        return self.sac.select_action(obs, deterministic)

    def save(self, path):
        self.sac.save(path)

    # ------------------------------------------------------------------ model
    def _xy(self, idx):
        s, a, r, sp, _ = self.real.gather(idx)
        return torch.cat([s, a], 1), torch.cat([sp - s, r[:, None]], 1)

    def train_model(self, epochs: int = None):
        c = self.cfg
        n = self.real.size
        perm = torch.randperm(n, device=self.device, generator=self.gen)
        nh = min(int(n * c.holdout_fraction), 5000)
        hold, train = perm[:nh], perm[nh:]
        x, y = self._xy(train)
        self.model.fit_scaler(x)
        nt, K = x.shape[0], c.ensemble
        loss = torch.zeros((), device=self.device)
        for _ in range(epochs or c.model_epochs):
            boot = torch.randint(0, nt, (nt, K), device=self.device, generator=self.gen)     # a bootstrap resample per member
            for b0 in range(0, nt, c.model_batch):
                ib = boot[b0: b0 + c.model_batch]
                mean, lv = self.model.forward(x[ib])
                loss, dm, dl = self.model.nll(mean, lv, y[ib])
                self.model.vjp(dm, dl)
                self.model_opt.step(zero_grad=True)
        with torch.no_grad():
            xh, yh = self._xy(hold) if nh else (x, y)
            mean, _ = self.model.forward(xh)
            mse = ((mean - yh[:, None]) ** 2).mean((0, 2))                                    # per member
            self.model.elite_idx = torch.argsort(mse)[: c.elites]
            self.holdout_mse = mse
        self.metrics.update(model_loss=loss, holdout_mse=mse[self.model.elite_idx].mean())
        return mse

    @torch.no_grad()
    def rollout_model(self):
        c = self.cfg
        s = self.real.gather(self.real.uniform_indices(c.rollout_batch))[0]
        for _ in range(c.rollout_len):
            a = self.sac.select_action(s).float()
            sp, r = self.model.predict(s, a, self.gen)
            d = self.termination_fn(s, a, sp).float()
            self.imagined.store_batch(s, a, r, sp, d)
            keep = d < 0.5
            if not bool(keep.any()):
                break
            s = sp[keep]

    # ------------------------------------------------------------------ policy
    def update(self, *unused):
        c = self.cfg
        n_real = max(int(c.batch * c.real_ratio), 1) if self.imagined.size else c.batch
        parts = [self.real.sample(n_real)]
        if c.batch - n_real > 0:
            parts.append(self.imagined.sample(c.batch - n_real))
        batch = [torch.cat([p[i] for p in parts]) for i in range(5)]
        self.sac.update(*batch)
        self.metrics.update(self.sac.metrics)
        return self.metrics


def run_mbpo(env, trainer: MBPOTrainer, total_env_steps: int, learning_starts: int = 1000, log_every: int = 0):
    """Uniform-random actions until ``learning_starts``; from then on the ensemble is refitted every ``model_train_every``
    env steps, followed by a batch of model rollouts; ``updates_per_step`` SAC updates follow each (batched) env step.
    Returns the list of finished episode returns."""
    c, dev = trainer.cfg, trainer.device
    obs = env.reset_batch().float().clone()
    ep_ret = torch.zeros(env.n_envs, device=dev)
    finished, step, next_fit = [], 0, learning_starts
    while step < total_env_steps:
        if step < learning_starts:
            a = torch.rand(env.n_envs, c.act_dim, device=dev) * 2 - 1
        else:
            a = trainer.select_action(obs).float()
        nxt, r, done, term = env.step_batch(a * 1.0)
        trainer.real.store_batch(obs, a, r.float(), env.next_obs.float(), term.float())
        ep_ret += r
        if bool(done.any()):
            finished.extend(ep_ret[done.bool()].tolist())
            ep_ret[done.bool()] = 0
        obs = nxt.float().clone()
        step += env.n_envs
        if step >= next_fit:
            trainer.train_model()
            next_fit += c.model_train_every
        if step >= learning_starts:
            trainer.rollout_model()
            for _ in range(c.updates_per_step):
                trainer.update()
        if log_every and step % log_every < env.n_envs:
            print(f"[mbpo] step {step} episodes {len(finished)} last {finished[-1] if finished else float('nan'):.1f}")
    return finished
