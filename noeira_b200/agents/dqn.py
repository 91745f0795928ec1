"""Value-based agents for discrete actions: DQN with double-Q targets, optional dueling head and n-step returns.

The Q-network is an ``nn.Sequential`` with explicit backward; the TD loss is the Huber loss on ``Q(s,a) − y`` with
``y = r + γⁿ (1 − d) Q_target(s', argmax_a Q(s', a))``; the target network follows by hard copy every
``target_every`` updates or by Polyak averaging when ``tau > 0``.
(Reference: noeira/deep_agents/dqn/ — DQNAgent / DQNTrainer / DQNConfig; the C51 / Rainbow variants are not built.)
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import nn


@dataclass
class DQNConfig:
    obs_dim: int = 4
    n_actions: int = 2
    hidden: int = 128
    batch: int = 128
    lr: float = 1e-3
    gamma: float = 0.99
    double_q: bool = True
    dueling: bool = False
    target_every: int = 200
    tau: float = 0.0
    eps_start: float = 1.0
    eps_end: float = 0.05
    eps_decay_steps: int = 5000
    huber_delta: float = 1.0
    max_grad_norm: float = 10.0
    seed: int = 0


class _DuelingHead(nn.Module):
    """Q = V + A − mean(A)."""

    def __init__(self, hidden, n_actions):
        super().__init__()
        self.v = self.add_child("value", nn.Linear(hidden, 1, out_fp32=True))
        self.a = self.add_child("advantage", nn.Linear(hidden, n_actions, out_fp32=True))

    def forward(self, h):
        v, a = self.v.forward(h).float(), self.a.forward(h).float()
        return v + a - a.mean(1, keepdim=True)

    def vjp(self, dq):
        dq = dq.float()
        dv = dq.sum(1, keepdim=True)
        da = dq - dq.mean(1, keepdim=True)
        return self.v.vjp(dv) + self.a.vjp(da)


def make_q_network(cfg: DQNConfig):
    trunk = [nn.LinearReLU(cfg.obs_dim, cfg.hidden, need_input_grad=False), nn.LinearReLU(cfg.hidden, cfg.hidden)]
    head = _DuelingHead(cfg.hidden, cfg.n_actions) if cfg.dueling else nn.Linear(cfg.hidden, cfg.n_actions, out_fp32=True)
    return nn.Sequential(*trunk, head)


class DQNTrainer:
    def __init__(self, cfg: DQNConfig = None, device="cpu"):
        self.cfg = cfg = cfg or DQNConfig()
        self.device = torch.device(device)
        nn.manual_seed(cfg.seed)
        self.q = make_q_network(cfg).to(self.device)
        self.q_target = make_q_network(cfg).to(self.device)
        self.q_target.copy_from(self.q)
        self.opt = nn.Adam(self.q.named_params(), lr=cfg.lr)
        self.opt.max_grad_norm = cfg.max_grad_norm
        self.gen = torch.Generator(device=self.device).manual_seed(cfg.seed + 1)
        self.updates = 0
        self.env_steps = 0

    def epsilon(self):
        c = self.cfg
        f = min(1.0, self.env_steps / max(c.eps_decay_steps, 1))
        return c.eps_start + f * (c.eps_end - c.eps_start)

    def _in(self, obs):
        return obs.to(torch.bfloat16) if self.device.type == "cuda" else obs.float()

    @torch.no_grad()
    def select_action(self, obs, explore=True):
        q = self.q.forward(self._in(obs)).float()
        a = q.argmax(1)
        if explore:
            n = obs.shape[0]
            rnd = torch.randint(0, self.cfg.n_actions, (n,), device=self.device, generator=self.gen)
            pick = torch.rand(n, device=self.device, generator=self.gen) < self.epsilon()
            a = torch.where(pick, rnd, a)
            self.env_steps += n
        return a

    def update(self, s, a, r, sp, d, n_step: int = 1):
        c, B = self.cfg, s.shape[0]
        with torch.no_grad():
            qn_t = self.q_target.forward(self._in(sp)).float()
            if c.double_q:
                sel = self.q.forward(self._in(sp)).float().argmax(1, keepdim=True)
                nxt = qn_t.gather(1, sel)[:, 0]
            else:
                nxt = qn_t.max(1).values
            y = r + (c.gamma ** n_step) * (1 - d) * nxt
        q = self.q.forward(self._in(s)).float()
        qa = q.gather(1, a.long()[:, None])[:, 0]
        diff = qa - y
        absd = diff.abs()
        loss = torch.where(absd <= c.huber_delta, 0.5 * diff * diff, c.huber_delta * (absd - 0.5 * c.huber_delta)).mean()
        dqa = diff.clamp(-c.huber_delta, c.huber_delta) / B
        dq = torch.zeros_like(q)
        dq.scatter_(1, a.long()[:, None], dqa[:, None])
        self.q.vjp(dq)
        if c.max_grad_norm > 0:
            self.opt.clip()
        self.opt.step(zero_grad=True)
        self.updates += 1
        if c.tau > 0:
            self.q_target.polyak_from(self.q, c.tau)
        elif self.updates % c.target_every == 0:
            self.q_target.copy_from(self.q)
        return dict(loss=loss, mean_q=qa.mean())
