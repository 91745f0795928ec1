"""MuZero-style agent on the batched tree search (planners/mcts.py).

Three networks — representation h(obs) → latent (min-max scaled to [0, 1]), dynamics g(latent, action) → (latent',
reward), prediction f(latent) → (policy logits, value) — trained on K-step unrolls of stored trajectories against the
search's visit-count policies, n-step value targets and observed rewards.  The networks are explicit-VJP modules
without a tape, and one module is applied K times inside an unroll, so the backward pass re-runs each step's forward
from its stored input and calls ``vjp`` right behind it (activation recomputation: one extra forward per step, no
stale caches).  Acting: one root-parallel MCTS per environment step over all environments at once.
Reference: noeira/deep_agents/muzero/ (agent, gpu_mcts orchestration, unrolled loss), noeira/planners/tree_search/.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from .. import nn
from ..planners.mcts import BatchedMCTS, MCTSConfig


@dataclass
class MuZeroConfig:
    obs_dim: int = 4
    n_actions: int = 2
    latent: int = 32
    hidden: int = 64
    n_simulations: int = 16
    discount: float = 0.997
    unroll: int = 4
    td_steps: int = 8
    batch: int = 128
    lr: float = 2e-3
    value_coef: float = 0.25
    reward_coef: float = 1.0
    window: int = 512              # steps kept per environment
    root_noise_frac: float = 0.25
    temperature: float = 1.0
    max_grad_norm: float = 5.0
    seed: int = 0
    # EfficientZero-style options: Gumbel root search with sequential halving (acting and policy targets), and a
    # self-supervised consistency loss −cos(ĥ_{t+k}, sg(h(o_{t+k}))) that ties the unrolled latents to the encoder
    gumbel: bool = False
    consistency_coef: float = 0.0


def _mlp(i, h, o):
    return nn.Sequential(nn.LinearTanh(i, h), nn.LinearTanh(h, h), nn.Linear(h, o, out_fp32=True))


def _scale01(x):
    lo, hi = x.min(-1, keepdim=True).values, x.max(-1, keepdim=True).values
    return (x - lo) / (hi - lo).clamp(min=1e-5)


def _scale01_vjp(x, dy):
    """Gradient of ``_scale01`` w.r.t. x (the two extreme elements carry the gradient of the range)."""
    lo, hi = x.min(-1, keepdim=True), x.max(-1, keepdim=True)
    span = (hi.values - lo.values).clamp(min=1e-5)
    y = (x - lo.values) / span
    dx = dy / span
    dlo = (-dy / span + dy * y / span).sum(-1, keepdim=True)     # d/dlo of (x - lo)/(hi - lo)
    dhi = (-dy * y / span).sum(-1, keepdim=True)
    dx.scatter_add_(-1, lo.indices, dlo)
    dx.scatter_add_(-1, hi.indices, dhi)
    return dx


class MuZeroAgent:
    def __init__(self, cfg: MuZeroConfig = None, n_envs: int = 16, device="cpu"):
        self.cfg = c = cfg or MuZeroConfig()
        self.device, self.n_envs = torch.device(device), n_envs
        nn.manual_seed(c.seed)
        self.repr = _mlp(c.obs_dim, c.hidden, c.latent).to(self.device)
        self.dyn = _mlp(c.latent + c.n_actions, c.hidden, c.latent + 1).to(self.device)
        self.pred = _mlp(c.latent, c.hidden, c.n_actions + 1).to(self.device)
        self.opt = nn.Adam(list(self.repr.named_params("repr.")) + list(self.dyn.named_params("dyn.")) +
                           list(self.pred.named_params("pred.")), lr=c.lr)
        self.opt.max_grad_norm = c.max_grad_norm
        self.gen = torch.Generator(device=self.device).manual_seed(c.seed + 1)
        self.mcts = BatchedMCTS(MCTSConfig(n_actions=c.n_actions, n_simulations=c.n_simulations, discount=c.discount,
                                           root_noise_frac=c.root_noise_frac, max_depth=c.n_simulations),
                                self._initial, self._recurrent)
        W, N = c.window, n_envs
        z = dict(device=self.device)
        self.obs_buf = torch.zeros(W, N, c.obs_dim, **z)
        self.act_buf = torch.zeros(W, N, dtype=torch.long, **z)
        self.rew_buf = torch.zeros(W, N, **z)
        self.done_buf = torch.zeros(W, N, **z)
        self.pol_buf = torch.zeros(W, N, c.n_actions, **z)
        self.val_buf = torch.zeros(W, N, **z)
        self.t = 0
        self.last: Dict[str, float] = {}
        self._pending = None

    def _inp(self, x):
        return x.to(torch.bfloat16) if self.device.type == "cuda" else x.float()

    # ---- model functions of the search
    def _initial(self, obs):
        h = _scale01(self.repr.forward(self._inp(obs)).float())
        out = self.pred.forward(self._inp(h)).float()
        return h, out[:, :-1], out[:, -1]

    def _recurrent(self, latent, action):
        c = self.cfg
        x = torch.cat([latent, torch.nn.functional.one_hot(action, c.n_actions).float()], dim=1)
        y = self.dyn.forward(self._inp(x)).float()
        h = _scale01(y[:, : c.latent])
        out = self.pred.forward(self._inp(h)).float()
        return h, y[:, c.latent], out[:, :-1], out[:, -1]

    # ---- step-wise interface of the generic on-policy driver
    @torch.no_grad()
    def select_action_batched(self, obs, greedy: bool = False):
        if self.cfg.gumbel:
            policy, value, action = self.mcts.search_gumbel(obs.to(self.device), generator=self.gen, greedy=greedy)
        else:
            policy, value, action = self.mcts.search(obs.to(self.device), temperature=0.0 if greedy else self.cfg.temperature,
                                                     generator=self.gen)
        self._pending = (policy, value)
        return action

    def record_batch(self, obs, action, reward, next_obs, done, terminated):
        i = self.t % self.cfg.window
        policy, value = self._pending
        self.obs_buf[i], self.act_buf[i], self.rew_buf[i], self.done_buf[i] = obs, action, reward, done
        self.pol_buf[i], self.val_buf[i] = policy, value
        self.t += 1

    # ---- training
    def _targets(self, idx_t, idx_e):
        """n-step value targets at positions (t, env) of the ring: Σ γ^i r_{t+i} + γ^n v_{t+n}, cut at episode ends and at
        the newest stored step."""
        c, W = self.cfg, self.cfg.window
        z = torch.zeros(len(idx_t), device=self.device)
        alive = torch.ones_like(z)
        disc = torch.ones_like(z)
        newest = self.t - 1
        for i in range(c.td_steps):
            tt = idx_t + i
            ok = (tt <= newest).float() * alive
            z = z + disc * ok * self.rew_buf[tt % W, idx_e]
            alive = ok * (1 - self.done_buf[tt % W, idx_e])
            disc = disc * c.discount
        tt = idx_t + c.td_steps
        boot = (tt <= newest).float() * alive
        return z + disc * boot * self.val_buf[tt % W, idx_e]

    def train_step(self) -> Optional[Dict[str, float]]:
        c, W = self.cfg, self.cfg.window
        have = min(self.t, W)
        if have < c.unroll + c.td_steps + 2 or self.t % 4 != 0:
            return None
        B = c.batch
        oldest = self.t - have
        t0 = torch.randint(oldest, self.t - c.unroll, (B,), device=self.device, generator=self.gen)
        e = torch.randint(0, self.n_envs, (B,), device=self.device, generator=self.gen)
        K = c.unroll
        # forward unroll, keeping each step's INPUT for the recomputing backward
        obs = self.obs_buf[t0 % W, e]
        raw0 = self.repr.forward(self._inp(obs)).float()
        h = _scale01(raw0)
        hs, raws, acts, alive_k = [h], [raw0], [], []
        alive = torch.ones(B, device=self.device)
        dpred, dhead = [], []
        dcons = [None] * (K + 1)
        loss_p = loss_v = loss_r = loss_c = 0.0
        for k in range(K + 1):
            tt = t0 + k
            out = self.pred.forward(self._inp(hs[k])).float()
            logits, v = out[:, :-1], out[:, -1]
            pi = self.pol_buf[tt % W, e]
            z = self._targets(tt, e)
            logp = torch.log_softmax(logits, -1)
            w = alive / (B * (K + 1))
            loss_p = loss_p - (w * (pi * logp).sum(-1)).sum()
            loss_v = loss_v + (w * (v - z).pow(2)).sum()
            dlogits = w[:, None] * (torch.softmax(logits, -1) * pi.sum(-1, keepdim=True) - pi)
            dv = c.value_coef * 2.0 * w * (v - z)
            dpred.append(torch.cat([dlogits, dv[:, None]], dim=1))
            if k == K:
                break
            a = self.act_buf[tt % W, e]
            x = torch.cat([hs[k], torch.nn.functional.one_hot(a, c.n_actions).float()], dim=1)
            y = self.dyn.forward(self._inp(x)).float()
            r_pred = y[:, c.latent]
            r_true = self.rew_buf[tt % W, e]
            loss_r = loss_r + (w * (r_pred - r_true).pow(2)).sum()
            dhead.append(c.reward_coef * 2.0 * w * (r_pred - r_true))
            raws.append(y[:, : c.latent])
            hs.append(_scale01(y[:, : c.latent]))
            if c.consistency_coef > 0:
                with torch.no_grad():
                    tgt = _scale01(self.repr.forward(self._inp(self.obs_buf[(tt + 1) % W, e])).float())
                hk = hs[-1].detach().requires_grad_(True)
                wn = alive * (1 - self.done_buf[tt % W, e]) / (B * K)
                with torch.enable_grad():
                    lc = -(wn * torch.nn.functional.cosine_similarity(hk, tgt, dim=-1)).sum()
                    lc.backward()
                dcons[k + 1] = c.consistency_coef * hk.grad
                loss_c = loss_c + float(lc.detach())
            acts.append(x)
            alive_k.append(alive)
            alive = alive * (1 - self.done_buf[tt % W, e])      # no targets past an episode end
        # backward with recomputation, last step first
        dh = torch.zeros(B, c.latent, device=self.device)
        for k in range(K, -1, -1):
            self.pred.forward(self._inp(hs[k]))
            dh = dh + self.pred.vjp(dpred[k]).float()
            if dcons[k] is not None:
                dh = dh + dcons[k]
            if k == 0:
                break
            # hs[k] = scale01(raws[k]), raws[k] = dyn(x_{k-1})[:, :latent]; the gradient is halved at every step so that
            # deep unrolls do not dominate the dynamics' update (as in the published algorithm)
            draw = _scale01_vjp(raws[k], dh) * 0.5
            self.dyn.forward(self._inp(acts[k - 1]))
            dx = self.dyn.vjp(torch.cat([draw, dhead[k - 1][:, None]], dim=1)).float()
            dh = dx[:, : c.latent]
        self.repr.forward(self._inp(obs))
        self.repr.vjp(_scale01_vjp(raw0, dh))
        if c.max_grad_norm > 0:
            self.opt.clip()
        self.opt.step(zero_grad=True)
        self.last = dict(policy_loss=float(loss_p), value_loss=float(loss_v), reward_loss=float(loss_r), consistency=float(loss_c))
        return self.last

    def save(self, path):
        from ..io.checkpoint import save_checkpoint
        save_checkpoint(path, list(self.repr.named_params("repr.")) + list(self.dyn.named_params("dyn.")) +
                        list(self.pred.named_params("pred.")), [], {f"opt.{k}": v for k, v in self.opt.scalars().items()})
