"""Discrete-action agents beyond DQN: C51 (categorical distributional Q), A2C and PPO with a categorical policy.

All three use ``nn.Sequential`` networks with explicit backward passes; the loss gradients with respect to the network
outputs are written out (no tape) and checked against autograd in the tests.

  C51Trainer          Q as a categorical distribution over ``n_atoms`` fixed supports in [v_min, v_max]; the target
                      distribution r + γⁿ z is projected back onto the support (Bellemare et al.), loss = cross entropy;
                      double-Q action selection on the expected value (noeira/deep_agents/c51/)
  A2CTrainer          synchronous advantage actor-critic over a batched env: n-step returns bootstrapped from V(s_T),
                      loss = −A·log π − c_ent·H + c_v·(V − R)² (noeira/deep_agents/a2c/)
  PPODiscreteTrainer  clipped-surrogate PPO with a categorical head, GAE(λ), minibatch epochs, per-minibatch advantage
                      normalisation (noeira/deep_agents/ppo_discrete/)
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import nn


def _mlp(i, h, o, need_in=False):
    return nn.Sequential(nn.LinearTanh(i, h, need_input_grad=need_in), nn.LinearTanh(h, h), nn.Linear(h, o, out_fp32=True))


def _inp(x, device):
    return x.to(torch.bfloat16) if device.type == "cuda" else x.float()


# ------------------------------------------------------------------------------------------ C51
@dataclass
class C51Config:
    obs_dim: int = 4
    n_actions: int = 2
    hidden: int = 128
    n_atoms: int = 51
    v_min: float = -10.0
    v_max: float = 10.0
    batch: int = 128
    lr: float = 1e-3
    gamma: float = 0.99
    target_every: int = 200
    eps_start: float = 1.0
    eps_end: float = 0.05
    eps_decay_steps: int = 5000
    max_grad_norm: float = 10.0
    seed: int = 0


def project_distribution(next_probs, r, d, support, gamma_n):
    """Categorical projection: mass of atom z_j at Tz_j = clamp(r + γⁿ(1−d) z_j) is split between its two neighbours on
    the support.  next_probs [B, N] → target probabilities [B, N]."""
    B, N = next_probs.shape
    v_min, v_max = float(support[0]), float(support[-1])
    dz = (v_max - v_min) / (N - 1)
    tz = (r[:, None] + gamma_n * (1 - d)[:, None] * support[None]).clamp(v_min, v_max)
    b = (tz - v_min) / dz
    lo, hi = b.floor().long(), b.ceil().long()
    same = (lo == hi).to(next_probs.dtype)                     # Tz exactly on an atom: all mass there
    out = torch.zeros_like(next_probs)
    out.scatter_add_(1, lo, next_probs * (hi.to(b.dtype) - b + same))
    out.scatter_add_(1, hi, next_probs * (b - lo.to(b.dtype)))
    return out


class C51Trainer:
    def __init__(self, cfg: C51Config = None, device="cpu"):
        self.cfg = cfg = cfg or C51Config()
        self.device = torch.device(device)
        nn.manual_seed(cfg.seed)
        mk = lambda: nn.Sequential(nn.LinearReLU(cfg.obs_dim, cfg.hidden, need_input_grad=False), nn.LinearReLU(cfg.hidden, cfg.hidden),
                                   nn.Linear(cfg.hidden, cfg.n_actions * cfg.n_atoms, out_fp32=True)).to(self.device)
        self.q, self.q_target = mk(), mk()
        self.q_target.copy_from(self.q)
        self.opt = nn.Adam(self.q.named_params(), lr=cfg.lr)
        self.opt.max_grad_norm = cfg.max_grad_norm
        self.support = torch.linspace(cfg.v_min, cfg.v_max, cfg.n_atoms, device=self.device)
        self.gen = torch.Generator(device=self.device).manual_seed(cfg.seed + 1)
        self.updates = self.env_steps = 0

    def _dist(self, net, obs):
        c = self.cfg
        return net.forward(_inp(obs, self.device)).float().reshape(-1, c.n_actions, c.n_atoms)

    def q_values(self, obs):
        return (torch.softmax(self._dist(self.q, obs), -1) * self.support).sum(-1)

    def epsilon(self):
        c = self.cfg
        return c.eps_start + min(1.0, self.env_steps / max(c.eps_decay_steps, 1)) * (c.eps_end - c.eps_start)

    @torch.no_grad()
    def select_action(self, obs, explore=True):
        a = self.q_values(obs).argmax(1)
        if explore:
            n = obs.shape[0]
            rnd = torch.randint(0, self.cfg.n_actions, (n,), device=self.device, generator=self.gen)
            a = torch.where(torch.rand(n, device=self.device, generator=self.gen) < self.epsilon(), rnd, a)
            self.env_steps += n
        return a

    def update(self, s, a, r, sp, d, n_step: int = 1):
        c, B = self.cfg, s.shape[0]
        with torch.no_grad():
            sel = self.q_values(sp).argmax(1)                                        # double Q: online net chooses
            nxt = torch.softmax(self._dist(self.q_target, sp), -1)[torch.arange(B), sel]
            target = project_distribution(nxt, r.float(), d.float(), self.support, c.gamma ** n_step)
        logits = self._dist(self.q, s)
        la = logits[torch.arange(B), a.long()]
        logp = torch.log_softmax(la, -1)
        loss = -(target * logp).sum(-1).mean()
        dlog = torch.zeros_like(logits)
        dlog[torch.arange(B), a.long()] = (logp.exp() - target) / B
        self.q.vjp(dlog.reshape(B, -1))
        if c.max_grad_norm > 0:
            self.opt.clip()
        self.opt.step(zero_grad=True)
        self.updates += 1
        if self.updates % c.target_every == 0:
            self.q_target.copy_from(self.q)
        return dict(loss=loss, mean_q=(logp.exp() * self.support).sum(-1).mean())


# ------------------------------------------------------------------------------------------ categorical policy math
def categorical_logp_entropy(logits, actions):
    logp_all = torch.log_softmax(logits.float(), -1)
    p = logp_all.exp()
    return logp_all.gather(1, actions.long()[:, None])[:, 0], -(p * logp_all).sum(-1), p, logp_all


def d_logp_d_logits(p, actions):
    return torch.nn.functional.one_hot(actions.long(), p.shape[1]).to(p.dtype) - p


def d_entropy_d_logits(p, logp_all, ent):
    return -p * (logp_all + ent[:, None])


# ------------------------------------------------------------------------------------------ A2C
@dataclass
class A2CConfig:
    obs_dim: int = 4
    n_actions: int = 2
    hidden: int = 64
    n_steps: int = 8
    lr: float = 7e-4
    gamma: float = 0.99
    value_coef: float = 0.5
    entropy_coef: float = 0.01
    max_grad_norm: float = 0.5
    seed: int = 0


class A2CTrainer:
    """Step-wise on-policy interface (``select_action_batched`` / ``record_batch`` / ``train_step``) of the generic
    driver ``training.rl.run_onpolicy_train_batched``."""

    def __init__(self, cfg: A2CConfig = None, n_envs: int = 16, device="cpu"):
        self.cfg = cfg = cfg or A2CConfig()
        self.device, self.n_envs = torch.device(device), n_envs
        nn.manual_seed(cfg.seed)
        self.actor = _mlp(cfg.obs_dim, cfg.hidden, cfg.n_actions).to(self.device)
        self.critic = _mlp(cfg.obs_dim, cfg.hidden, 1).to(self.device)
        self.opt = nn.Adam(list(self.actor.named_params("actor.")) + list(self.critic.named_params("critic.")), lr=cfg.lr)
        self.opt.max_grad_norm = cfg.max_grad_norm
        self.gen = torch.Generator(device=self.device).manual_seed(cfg.seed + 1)
        self.buf = []
        self.last = {}

    @torch.no_grad()
    def select_action_batched(self, obs, greedy=False):
        logits = self.actor.forward(_inp(obs, self.device)).float()
        if greedy:
            return logits.argmax(1)
        return torch.multinomial(torch.softmax(logits, -1), 1, generator=self.gen)[:, 0]

    def record_batch(self, obs, action, reward, next_obs, done, terminated):
        self.buf.append((obs.clone(), action.clone(), reward.clone(), next_obs.clone(), done.clone(), terminated.clone()))

    def train_step(self):
        c = self.cfg
        if len(self.buf) < c.n_steps:
            return None
        T, N = len(self.buf), self.n_envs
        obs = torch.stack([b[0] for b in self.buf])
        act = torch.stack([b[1] for b in self.buf])
        rew = torch.stack([b[2] for b in self.buf]).float()
        nobs = torch.stack([b[3] for b in self.buf])
        done = torch.stack([b[4] for b in self.buf]).float()
        term = torch.stack([b[5] for b in self.buf]).float()
        self.buf = []
        with torch.no_grad():
            vnext = self.critic.forward(_inp(nobs.reshape(T * N, -1), self.device)).float().reshape(T, N)
            ret = torch.zeros(T, N, device=self.device)
            run = vnext[-1] * (1 - term[-1])
            for t in range(T - 1, -1, -1):
                # an episode that ended at t bootstraps from its own final state (zero when terminated)
                run = torch.where(done[t] > 0.5, (1 - term[t]) * vnext[t], run)
                run = rew[t] + c.gamma * run
                ret[t] = run
        flat_obs, flat_act, flat_ret = obs.reshape(T * N, -1), act.reshape(-1), ret.reshape(-1)
        B = T * N
        logits = self.actor.forward(_inp(flat_obs, self.device)).float()
        v = self.critic.forward(_inp(flat_obs, self.device)).float()[:, 0]
        logp, ent, p, logp_all = categorical_logp_entropy(logits, flat_act)
        adv = (flat_ret - v).detach()
        pol_loss, v_loss = -(adv * logp).mean(), (v - flat_ret).pow(2).mean()
        dlogits = (-(adv / B)[:, None] * d_logp_d_logits(p, flat_act) - c.entropy_coef / B * d_entropy_d_logits(p, logp_all, ent))
        dv = c.value_coef * 2.0 * (v - flat_ret) / B
        self.actor.vjp(dlogits)
        self.critic.vjp(dv[:, None])
        if c.max_grad_norm > 0:
            self.opt.clip()
        self.opt.step(zero_grad=True)
        self.last = dict(policy_loss=float(pol_loss), value_loss=float(v_loss), entropy=float(ent.mean()))
        return self.last

    def save(self, path):
        from ..io.checkpoint import save_checkpoint
        save_checkpoint(path, list(self.actor.named_params("actor.")) + list(self.critic.named_params("critic.")), [],
                        {f"opt.{k}": v for k, v in self.opt.scalars().items()})


# ------------------------------------------------------------------------------------------ PPO (discrete)
@dataclass
class PPODiscreteConfig:
    obs_dim: int = 4
    n_actions: int = 2
    hidden: int = 64
    rollout_len: int = 32
    n_epochs: int = 4
    n_minibatches: int = 4
    lr: float = 3e-4
    gamma: float = 0.99
    gae_lambda: float = 0.95
    clip_eps: float = 0.2
    value_coef: float = 0.5
    entropy_coef: float = 0.01
    max_grad_norm: float = 0.5
    seed: int = 0


def ppo_discrete_objective(logits, actions, old_logp, adv, clip_eps, entropy_coef):
    """Clipped surrogate with a categorical policy; returns (loss, dL/dlogits, approx KL, clip fraction)."""
    B = logits.shape[0]
    logp, ent, p, logp_all = categorical_logp_entropy(logits, actions)
    diff = (logp - old_logp).clamp(-20, 20)
    ratio = diff.exp()
    s1, s2 = ratio * adv, ratio.clamp(1 - clip_eps, 1 + clip_eps) * adv
    loss = -torch.minimum(s1, s2).mean() - entropy_coef * ent.mean()
    # the clipped branch is flat in the ratio where it is active
    use1 = (s1 <= s2) | ((ratio >= 1 - clip_eps) & (ratio <= 1 + clip_eps))
    dlogp = -(adv * ratio * use1.to(adv.dtype)) / B
    dlogits = dlogp[:, None] * d_logp_d_logits(p, actions) - entropy_coef / B * d_entropy_d_logits(p, logp_all, ent)
    clipped = ((ratio - 1).abs() > clip_eps).float().mean()
    return loss, dlogits, (-diff).mean(), clipped


class PPODiscreteTrainer(A2CTrainer):
    def __init__(self, cfg: PPODiscreteConfig = None, n_envs: int = 16, device="cpu"):
        self.cfg = cfg = cfg or PPODiscreteConfig()
        self.device, self.n_envs = torch.device(device), n_envs
        nn.manual_seed(cfg.seed)
        self.actor = _mlp(cfg.obs_dim, cfg.hidden, cfg.n_actions).to(self.device)
        self.critic = _mlp(cfg.obs_dim, cfg.hidden, 1).to(self.device)
        self.opt = nn.Adam(list(self.actor.named_params("actor.")) + list(self.critic.named_params("critic.")), lr=cfg.lr)
        self.opt.max_grad_norm = cfg.max_grad_norm
        self.gen = torch.Generator(device=self.device).manual_seed(cfg.seed + 1)
        self.buf, self.last = [], {}

    def train_step(self):
        c = self.cfg
        if len(self.buf) < c.rollout_len:
            return None
        T, N = len(self.buf), self.n_envs
        obs = torch.stack([b[0] for b in self.buf]).reshape(T * N, -1)
        act = torch.stack([b[1] for b in self.buf]).reshape(-1)
        rew = torch.stack([b[2] for b in self.buf]).float()
        nobs = torch.stack([b[3] for b in self.buf])
        done = torch.stack([b[4] for b in self.buf]).float()
        term = torch.stack([b[5] for b in self.buf]).float()
        self.buf = []
        with torch.no_grad():
            val = self.critic.forward(_inp(obs, self.device)).float().reshape(T, N)
            vnext = self.critic.forward(_inp(nobs.reshape(T * N, -1), self.device)).float().reshape(T, N)
            old_logp = categorical_logp_entropy(self.actor.forward(_inp(obs, self.device)), act)[0]
            adv = torch.zeros(T, N, device=self.device)
            gae = torch.zeros(N, device=self.device)
            for t in range(T - 1, -1, -1):
                boundary = (done[t] > 0.5) | (t == T - 1)
                nv = torch.where(boundary, (1 - term[t]) * vnext[t], val[min(t + 1, T - 1)])
                delta = rew[t] + c.gamma * nv - val[t]
                gae = delta + c.gamma * c.gae_lambda * (1 - done[t]) * gae
                adv[t] = gae
            ret = (adv + val).reshape(-1)
            adv = adv.reshape(-1)
        B = T * N
        mb = B // c.n_minibatches
        stats = []
        for _ in range(c.n_epochs):
            perm = torch.randperm(B, device=self.device, generator=self.gen)
            for k in range(c.n_minibatches):
                idx = perm[k * mb:(k + 1) * mb]
                a = adv[idx]
                a = (a - a.mean()) / (a.std(unbiased=False) + 1e-8)
                logits = self.actor.forward(_inp(obs[idx], self.device)).float()
                loss, dlogits, kl, cf = ppo_discrete_objective(logits, act[idx], old_logp[idx], a, c.clip_eps, c.entropy_coef)
                v = self.critic.forward(_inp(obs[idx], self.device)).float()[:, 0]
                self.actor.vjp(dlogits)
                self.critic.vjp((c.value_coef * 2.0 * (v - ret[idx]) / mb)[:, None])
                if c.max_grad_norm > 0:
                    self.opt.clip()
                self.opt.step(zero_grad=True)
                stats.append((float(loss), float((v - ret[idx]).pow(2).mean()), float(kl), float(cf)))
        s = torch.tensor(stats).mean(0).tolist()
        self.last = dict(policy_loss=s[0], value_loss=s[1], approx_kl=s[2], clip_frac=s[3])
        return self.last
