"""REDQ: SAC with an ensemble of N critics, targets from the minimum over a random subset of M of them, and a high
update-to-data ratio; the actor ascends the MEAN of all critics.  (Chen et al., "Randomized Ensembled Double
Q-Learning", 2021; reference: noeira/deep_agents/redq/.)  Same explicit-VJP pattern, distribution head, temperature
optimizer and replay interface as ``agents/sac.py``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import nn
from .sac import SquashedGaussian, make_critic, make_sac_actor


@dataclass
class REDQConfig:
    obs_dim: int = 17
    act_dim: int = 6
    hidden: int = 256
    n_critics: int = 10
    subset: int = 2
    utd: int = 20                  # critic updates per environment step; the actor is updated once, after the last
    batch: int = 256
    actor_lr: float = 3e-4
    critic_lr: float = 3e-4
    alpha_lr: float = 3e-4
    gamma: float = 0.99
    tau: float = 0.005
    init_alpha: float = 0.2
    action_scale: float = 1.0
    auto_entropy: bool = True
    seed: int = 0


class REDQTrainer:
    def __init__(self, cfg: REDQConfig = None, device="cpu"):
        self.cfg = c = cfg or REDQConfig()
        self.device = torch.device(device)
        nn.manual_seed(c.seed)
        O, A, H = c.obs_dim, c.act_dim, c.hidden
        self.actor = make_sac_actor(O, A, H).to(self.device)
        self.qs = [make_critic(O, A, H).to(self.device) for _ in range(c.n_critics)]
        self.qts = [make_critic(O, A, H).to(self.device) for _ in range(c.n_critics)]
        for q, t in zip(self.qs, self.qts):
            t.copy_from(q)
        self.actor_opt = nn.Adam(self.actor.named_params(), lr=c.actor_lr)
        named = [p for i, q in enumerate(self.qs) for p in q.named_params(f"q{i}.")]
        self.critic_opt = nn.Adam(named, lr=c.critic_lr)
        self.target_arena = nn.ParamArena([p for i, q in enumerate(self.qts) for p in q.named_params(f"q{i}.")], with_moments=False)
        self.alpha_opt = nn.ScalarAdam(c.init_alpha, c.alpha_lr, device=self.device)
        self.target_entropy = -float(A)
        self.dist = SquashedGaussian(A, c.action_scale)
        self.gen = torch.Generator(device=self.device).manual_seed(c.seed + 1)
        self.total_train_steps = 0
        self.metrics = {}

    def _in(self, x):
        if self.device.type == "cuda":
            w = (x.shape[1] + 7) // 8 * 8
            out = torch.zeros(x.shape[0], w, device=self.device, dtype=torch.bfloat16)
            out[:, : x.shape[1]] = x
            return out[:, : x.shape[1]]
        return x

    def _sa(self, s, a):
        return self._in(torch.cat([s.float(), a.float()], 1))

    def _noise(self, n):
        return torch.randn(n, self.cfg.act_dim, device=self.device, generator=self.gen)

    @property
    def alpha(self):
        return self.alpha_opt.alpha

    def select_action(self, obs, deterministic=False):
        packed = self.actor.forward(self._in(obs))
        if deterministic:
            return self.cfg.action_scale * torch.tanh(packed.float()[:, : self.cfg.act_dim])
        return self.dist.forward(packed, self._noise(obs.shape[0]))[0]

    def critic_update(self, s, a, r, sp, d):
        c = self.cfg
        B = s.shape[0]
        alpha = float(self.alpha) if self.device.type == "cpu" else self.alpha
        ap, logpp = self.dist.forward(self.actor.forward(self._in(sp)), self._noise(B))
        sap = self._sa(sp, ap)
        idx = torch.randperm(c.n_critics, generator=torch.Generator().manual_seed(c.seed + 7919 * self.total_train_steps))[: c.subset]
        qt = torch.stack([self.qts[int(i)].forward(sap).float()[:, 0] for i in idx]).min(0).values
        y = r + c.gamma * (1 - d) * (qt - alpha * logpp)
        sa = self._sa(s, a)
        loss = 0.0
        for q in self.qs:
            diff = q.forward(sa).float()[:, 0] - y
            loss = loss + (diff * diff).mean()
            q.vjp((2.0 / B * diff)[:, None])
        self.critic_opt.step(zero_grad=True)
        nn.polyak(self.target_arena, self.critic_opt.arena, c.tau)
        self.total_train_steps += 1
        return loss / c.n_critics

    def actor_update(self, s):
        c = self.cfg
        B = s.shape[0]
        alpha = float(self.alpha) if self.device.type == "cpu" else self.alpha
        packed = self.actor.forward(self._in(s))
        api, logpi = self.dist.forward(packed, self._noise(B))
        sapi = self._sa(s, api)
        ps = [p for q in self.qs for p in q.params()]
        for p in ps:
            p.frozen = True
        qmean, da = 0.0, 0.0
        for q in self.qs:
            qmean = qmean + q.forward(sapi).float()[:, 0] / c.n_critics
            da = da + q.vjp(torch.full((B, 1), -1.0 / (B * c.n_critics), device=self.device)).float()
        for p in ps:
            p.frozen = False
        da = da[:, c.obs_dim: c.obs_dim + c.act_dim]
        dpacked = self.dist.vjp(da, torch.full((B,), 1.0, device=self.device) * alpha / B)
        self.actor.vjp(dpacked if self.device.type == "cpu" else dpacked.to(torch.bfloat16))
        self.actor_opt.step(zero_grad=True)
        if c.auto_entropy:
            self.alpha_opt.step_alpha(logpi.mean().reshape(1) if self.device.type == "cuda" else logpi.mean(), self.target_entropy)
        return (alpha * logpi - qmean).mean(), qmean.mean(), logpi.mean()

    def update(self, s, a, r, sp, d):
        """One call of the generic off-policy driver = one critic update; every ``utd``-th call also updates the actor
        and the temperature (run the driver with ``utd=cfg.utd``)."""
        closs = self.critic_update(s, a, r, sp, d)
        if self.total_train_steps % self.cfg.utd == 0:
            aloss, mq, mlp = self.actor_update(s)
            self.metrics = dict(critic_loss=closs, actor_loss=aloss, mean_q=mq, mean_logp=mlp)
        else:
            self.metrics = dict(self.metrics, critic_loss=closs)
        return self.metrics

    def save(self, path):
        from ..io.checkpoint import save_checkpoint
        params = list(self.actor.named_params("actor.")) + [p for i, q in enumerate(self.qs) for p in q.named_params(f"q{i}.")]
        save_checkpoint(path, params, [], {"alpha": float(self.alpha), "steps": float(self.total_train_steps)})
