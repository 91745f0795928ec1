"""TD-MPC2: a decoder-free latent world model trained by temporal-difference learning, acted on by planning.

Components (all ``nn`` modules with explicit backward; the unrolled training graph applies them repeatedly through
``nn.apply``):

  encoder   h(s)      → z, simplicial normalisation (``simnorm``: softmax inside groups of ``simnorm_dim`` entries)
  dynamics  d(z, a)   → z'   (simnorm)
  reward    R(z, a)   → r
  Q         Q_k(z, a) for an ensemble of ``n_q`` critics evaluated as ONE ``nn.BlockLinear`` network
  prior     π(z)      → squashed Gaussian action

``train_step`` samples length-``horizon`` sub-sequences from the per-env ring, unrolls the dynamics from the encoded first
observation, and minimises Σ_t ρ^t [ consistency ‖z_{t+1} − sg(h(s_{t+1}))‖² + reward (R − r_t)² + value Σ_k (Q_k − y_t)² ]
with ``y_t = r_t + γ (1 − d) · min of two random target critics at (h(s_{t+1}), π(h(s_{t+1})))``; the prior maximises the
ensemble-mean Q of its own action (scaled by a running magnitude) plus an entropy bonus on detached latents; target
critics follow by Polyak averaging.  ``plan`` is MPPI in latent space for a whole batch of environments: sequences sampled
around a warm-started mean plus sequences proposed by the prior, scored by Σ γ^t R + γ^H · mean-Q at the end, the elite
set re-weights the mean / std for a few iterations, the executed action is drawn from the elites.
(noeira/deep_agents/tdmpc2/: world model, losses.mojo (mse / bce kernels), batched_acting.mojo greedy-action kernel;
multi-task variants batched_acting_mt.mojo are not built.)
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional

import torch

from .. import nn


@dataclass
class TDMPC2Config:
    obs_dim: int = 3
    act_dim: int = 1
    latent: int = 64
    simnorm_dim: int = 8
    hidden: int = 128
    n_q: int = 5
    horizon: int = 3
    batch: int = 128
    lr: float = 1e-3
    enc_lr_scale: float = 0.3
    gamma: float = 0.97
    rho: float = 0.5
    tau: float = 0.01
    consistency_coef: float = 20.0
    reward_coef: float = 0.5
    value_coef: float = 0.5
    entropy_coef: float = 1e-4
    max_grad_norm: float = 20.0
    log_std_min: float = -5.0
    log_std_max: float = 1.0
    # planning
    plan_samples: int = 128
    plan_pi_samples: int = 16
    plan_elites: int = 16
    plan_iterations: int = 3
    plan_max_std: float = 1.0
    plan_min_std: float = 0.05
    plan_temperature: float = 0.5
    window: int = 4096                 # ring length per env
    seed: int = 0


def simnorm(x, d):
    s = x.shape
    return torch.softmax(x.reshape(*s[:-1], s[-1] // d, d), -1).reshape(s)


def _mlp(i, h, o, first_needs_input_grad=True):
    return nn.Sequential(nn.Linear(i, h, act="silu", need_input_grad=first_needs_input_grad), nn.Linear(h, h, act="silu"),
                         nn.Linear(h, o, out_fp32=True))


class _QEnsemble(nn.Module):
    def __init__(self, i, h, k):
        super().__init__()
        self.net = self.add_child("net", nn.Sequential(nn.BlockLinear(i, h, k, act="silu"), nn.BlockLinear(h, h, k, act="silu"),
                                                       nn.BlockLinear(h, 1, k)))

    def forward(self, za):
        return self.net.forward(za).float()[..., 0]                     # [B, K]

    def vjp(self, dq):
        return self.net.vjp(dq[..., None])


class TDMPC2Agent:
    def __init__(self, cfg: TDMPC2Config = None, n_envs: int = 8, device="cpu"):
        self.cfg = c = cfg or TDMPC2Config()
        assert c.latent % c.simnorm_dim == 0
        self.device, self.n_envs = torch.device(device), n_envs
        nn.manual_seed(c.seed)
        L, A, H = c.latent, c.act_dim, c.hidden
        self.enc = _mlp(c.obs_dim, H, L, first_needs_input_grad=False).to(self.device)
        self.dyn = _mlp(L + A, H, L).to(self.device)
        self.rew = _mlp(L + A, H, 1).to(self.device)
        self.q, self.q_target = _QEnsemble(L + A, H, c.n_q).to(self.device), _QEnsemble(L + A, H, c.n_q).to(self.device)
        self.q_target.copy_from(self.q)
        self.pi = _mlp(L, H, 2 * A).to(self.device)
        self.opt = nn.Adam(list(self.enc.named_params("enc.")) + list(self.dyn.named_params("dyn.")) +
                           list(self.rew.named_params("rew.")) + list(self.q.named_params("q.")), lr=c.lr)
        self.opt.max_grad_norm = c.max_grad_norm
        self.pi_opt = nn.Adam(self.pi.named_params("pi."), lr=c.lr)
        self.pi_opt.max_grad_norm = c.max_grad_norm
        self.gen = torch.Generator(device=self.device).manual_seed(c.seed + 1)
        W, E = c.window, n_envs
        z = dict(device=self.device)
        self.obs_buf = torch.zeros(W, E, c.obs_dim, **z)
        self.next_buf = torch.zeros(W, E, c.obs_dim, **z)
        self.act_buf = torch.zeros(W, E, A, **z)
        self.rew_buf = torch.zeros(W, E, **z)
        self.term_buf = torch.zeros(W, E, **z)
        self.done_buf = torch.zeros(W, E, **z)
        self.t = 0
        self.q_scale = 1.0
        self._mean = torch.zeros(E, c.horizon, A, **z)
        self._fresh = torch.ones(E, dtype=torch.bool, device=self.device)
        self.last: Dict[str, float] = {}

    # ------------------------------------------------------------------ model pieces (plain tensors in, plain tensors out)
    def _x(self, t):
        return t.to(torch.bfloat16) if self.device.type == "cuda" else t.float()

    def encode(self, obs):
        return simnorm(self.enc.forward(self._x(obs)).float(), self.cfg.simnorm_dim)

    def next_latent(self, z, a):
        return simnorm(self.dyn.forward(self._x(torch.cat([z, a], -1))).float(), self.cfg.simnorm_dim)

    def reward(self, z, a):
        return self.rew.forward(self._x(torch.cat([z, a], -1))).float()[:, 0]

    def _pi_dist(self, out):
        c = self.cfg
        mu, ls = out[:, : c.act_dim], out[:, c.act_dim:]
        ls = c.log_std_min + 0.5 * (c.log_std_max - c.log_std_min) * (torch.tanh(ls) + 1)
        return mu, ls

    def policy(self, z, sample=True):
        mu, ls = self._pi_dist(self.pi.forward(self._x(z)).float())
        eps = torch.randn(mu.shape, device=self.device, generator=self.gen) if sample else torch.zeros_like(mu)
        return torch.tanh(mu + ls.exp() * eps)

    # ------------------------------------------------------------------ acting: batched MPPI in latent space
    @torch.no_grad()
    def _score(self, z, actions):
        """z [E·N, L], actions [E·N, H, A] → discounted model return plus terminal value."""
        c = self.cfg
        G, disc = torch.zeros(z.shape[0], device=self.device), 1.0
        for t in range(c.horizon):
            a = actions[:, t]
            G = G + disc * self.reward(z, a)
            z = self.next_latent(z, a)
            disc *= c.gamma
        q = self.q.forward(self._x(torch.cat([z, self.policy(z)], -1)))
        return G + disc * q.mean(1)

    @torch.no_grad()
    def plan(self, obs, explore=True):
        c, E = self.cfg, obs.shape[0]
        N, NP, H, A = c.plan_samples, c.plan_pi_samples, c.horizon, c.act_dim
        z0 = self.encode(obs)
        # warm start: last plan shifted by one step, zero for fresh episodes
        mean = torch.cat([self._mean[:, 1:], torch.zeros(E, 1, A, device=self.device)], 1)
        mean = torch.where(self._fresh[:, None, None], torch.zeros_like(mean), mean)
        std = torch.full((E, H, A), c.plan_max_std, device=self.device)
        pi_actions = torch.zeros(E, NP, H, A, device=self.device)
        if NP > 0:
            z = z0[:, None].expand(E, NP, -1).reshape(E * NP, -1)
            for t in range(H):
                a = self.policy(z)
                pi_actions[:, :, t] = a.reshape(E, NP, A)
                z = self.next_latent(z, a)
        zr = z0[:, None].expand(E, N, -1).reshape(E * N, -1)
        for _ in range(c.plan_iterations):
            noise = torch.randn(E, N - NP, H, A, device=self.device, generator=self.gen)
            acts = torch.cat([pi_actions, (mean[:, None] + std[:, None] * noise).clamp(-1, 1)], 1)       # [E, N, H, A]
            val = self._score(zr, acts.reshape(E * N, H, A)).reshape(E, N)
            top = val.topk(c.plan_elites, dim=1)
            elite = acts.gather(1, top.indices[:, :, None, None].expand(-1, -1, H, A))
            w = torch.softmax((top.values - top.values.max(1, keepdim=True).values) / c.plan_temperature, 1)[:, :, None, None]
            mean = (w * elite).sum(1)
            std = ((w * (elite - mean[:, None]) ** 2).sum(1)).sqrt().clamp(c.plan_min_std, c.plan_max_std)
        pick = torch.multinomial(w[:, :, 0, 0], 1, generator=self.gen)[:, 0]
        a = elite[torch.arange(E, device=self.device), pick, 0]
        if explore:
            a = (a + std[:, 0] * torch.randn(E, A, device=self.device, generator=self.gen)).clamp(-1, 1)
        self._mean, self.plan_value = mean, top.values[:, 0]
        self._fresh = torch.zeros_like(self._fresh)
        return a

    def select_action(self, obs, explore=True):
        return self.plan(obs.to(self.device).float(), explore)

    def record_batch(self, obs, action, reward, next_obs, done, terminated):
        i = self.t % self.cfg.window
        self.obs_buf[i], self.next_buf[i], self.act_buf[i] = obs, next_obs, action
        self.rew_buf[i], self.term_buf[i], self.done_buf[i] = reward, terminated, done
        self._fresh = self._fresh | done.bool()
        self.t += 1

    # ------------------------------------------------------------------ training
    def train_step(self) -> Optional[Dict[str, float]]:
        c, W = self.cfg, self.cfg.window
        have = min(self.t, W)
        H = c.horizon
        if have < H + 1:
            return None
        B, dev = c.batch, self.device
        t0 = torch.randint(self.t - have, self.t - H + 1, (B,), device=dev, generator=self.gen)
        e = torch.randint(0, self.n_envs, (B,), device=dev, generator=self.gen)
        # ---- targets (no gradient): encoded successors and TD targets from two random target critics
        with torch.no_grad():
            zn = [self.encode(self.next_buf[(t0 + t) % W, e]) for t in range(H)]
            k2 = torch.randperm(c.n_q, device=dev, generator=self.gen)[:2]
            ys = []
            for t in range(H):
                qn = self.q_target.forward(self._x(torch.cat([zn[t], self.policy(zn[t])], -1)))[:, k2].min(1).values
                ys.append(self.rew_buf[(t0 + t) % W, e] + c.gamma * (1 - self.term_buf[(t0 + t) % W, e]) * qn)
        # ---- unrolled model loss through the re-entrant bridge
        z = simnorm(nn.apply(self.enc, self._x(self.obs_buf[t0 % W, e])).float(), c.simnorm_dim)
        alive = torch.ones(B, device=dev)
        cons = rl = vl = 0.0
        zs = []
        for t in range(H):
            zs.append(z.detach())
            a = self.act_buf[(t0 + t) % W, e]
            za = torch.cat([z, a], -1)
            w = alive * (c.rho ** t) / B
            r = nn.apply(self.rew, self._x(za)).float()[:, 0]
            q = nn.apply(self.q, self._x(za))                                        # [B, K]
            z = simnorm(nn.apply(self.dyn, self._x(za)).float(), c.simnorm_dim)
            cons = cons + (w * (z - zn[t]).pow(2).mean(-1)).sum()
            rl = rl + (w * (r - self.rew_buf[(t0 + t) % W, e]).pow(2)).sum()
            vl = vl + (w[:, None] * (q - ys[t][:, None]).pow(2)).sum() / c.n_q
            alive = alive * (1 - self.done_buf[(t0 + t) % W, e])                     # nothing is learned across a reset
        loss = c.consistency_coef * cons + c.reward_coef * rl + c.value_coef * vl
        loss.backward()
        if c.max_grad_norm > 0:
            self.opt.clip()
        self.opt.step(zero_grad=True)
        # ---- policy prior on the detached latents of the unroll
        zc = torch.cat(zs, 0)
        out = nn.apply(self.pi, self._x(zc)).float()
        mu, ls = self._pi_dist(out)
        eps = torch.randn(mu.shape, device=dev, generator=self.gen)
        u = mu + ls.exp() * eps
        a = torch.tanh(u)
        logp = (-0.5 * eps.pow(2) - ls - 0.5 * math.log(2 * math.pi)).sum(-1) - torch.log(1 - a.pow(2) + 1e-6).sum(-1)
        qpi = nn.apply(self.q, self._x(torch.cat([zc, a], -1))).mean(1)
        self.q_scale = 0.99 * self.q_scale + 0.01 * float(qpi.detach().abs().mean().clamp(min=1.0))
        pl = (-(qpi / self.q_scale) + c.entropy_coef * logp).mean()
        pl.backward()
        if c.max_grad_norm > 0:
            self.pi_opt.clip()
        self.pi_opt.step(zero_grad=True)
        self.opt.arena.grd.zero_()                       # the critic's parameter gradients of the policy pass are not used
        self.q_target.polyak_from(self.q, c.tau)
        self.last = {k: float(v.detach()) for k, v in dict(consistency=cons, reward_loss=rl, value_loss=vl, policy_loss=pl,
                                                           q_mean=qpi.mean()).items()}
        return self.last

    def save(self, path):
        from ..io.checkpoint import save_checkpoint
        save_checkpoint(path, list(self.enc.named_params("enc.")) + list(self.dyn.named_params("dyn.")) +
                        list(self.rew.named_params("rew.")) + list(self.q.named_params("q.")) +
                        list(self.pi.named_params("pi.")), [], {"steps": float(self.t)})


def run_tdmpc2(env, agent: TDMPC2Agent, total_env_steps: int, seed_steps: int = 500, updates_per_step: int = 1):
    """Random actions for ``seed_steps`` env steps, then plan → step → record → update.  Returns finished episode returns."""
    dev, c = agent.device, agent.cfg
    obs = env.reset_batch().float().clone()
    ep_ret = torch.zeros(env.n_envs, device=dev)
    finished, step = [], 0
    while step < total_env_steps:
        if step < seed_steps:
            a = torch.rand(env.n_envs, c.act_dim, device=dev) * 2 - 1
        else:
            a = agent.select_action(obs)
        nxt, r, done, term = env.step_batch(a)
        agent.record_batch(obs, a, r.float(), env.next_obs.float(), done.float(), term.float())
        ep_ret += r
        if bool(done.any()):
            finished.extend(ep_ret[done.bool()].tolist())
            ep_ret[done.bool()] = 0
        obs = nxt.float().clone()
        step += env.n_envs
        if step >= seed_steps:
            for _ in range(updates_per_step):
                agent.train_step()
    return finished
