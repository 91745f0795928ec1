"""DreamerV3: a recurrent state-space world model with categorical latents, and an actor-critic trained in imagination.

World model (every network an ``nn`` module with explicit backward, applied once per time step through ``nn.apply``):

  encoder      e_t   = enc(symlog(o_t))
  sequence     h_t   = GRU(silu(W [z_{t-1}, a_{t-1}]), h_{t-1})            (state reset where an episode starts)
  prior        p(z_t | h_t),  posterior q(z_t | h_t, e_t): ``groups`` categoricals of ``classes`` classes, 1 % uniform mix,
               one-hot samples with straight-through gradients
  heads        decoder (symlog-MSE), reward (two-hot over symlog bins), continue (Bernoulli) on [h_t, z_t]
  loss         prediction + 0.5 · max(1, KL[sg(q) ‖ p]) + 0.1 · max(1, KL[q ‖ sg(p)])          (free bits)

Behaviour: from every posterior state of the batch the model is rolled forward ``imag_horizon`` steps with actions of the
actor; the critic (two-hot over symlog bins, EMA regulariser) learns λ-returns; the actor follows the gradient of the
λ-returns through the dynamics (continuous actions), scaled by the running 5–95 percentile range of the returns, plus an
entropy bonus.  World-model parameter gradients produced by the behaviour pass are discarded.
(noeira/deep_agents/dreamerv3/: rssm_ops.mojo — GRU, block-GRU action mix, straight-through sampling kernels;
onehot_kl.mojo — categorical KL with free bits; wm_loss_ops.mojo — symlog-MSE and Bernoulli heads.)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict

import torch
import torch.nn.functional as F

from .. import nn
from ..nn.losses import symexp, symlog, two_hot


@dataclass
class DreamerV3Config:
    obs_dim: int = 3
    act_dim: int = 1
    deter: int = 64
    groups: int = 8
    classes: int = 8
    hidden: int = 64
    bins: int = 41
    bin_range: float = 10.0            # symlog range covered by the two-hot bins
    seq_len: int = 16
    batch: int = 16
    imag_horizon: int = 8
    gamma: float = 0.97
    lam: float = 0.95
    lr: float = 1e-3
    ac_lr: float = 3e-4
    unimix: float = 0.01
    free_bits: float = 1.0
    beta_dyn: float = 0.5
    beta_rep: float = 0.1
    entropy_coef: float = 3e-4
    critic_ema: float = 0.98
    critic_reg: float = 1.0
    max_grad_norm: float = 100.0
    window: int = 2048
    seed: int = 0


def _mlp(i, h, o, need_in=True):
    return nn.Sequential(nn.Linear(i, h, act="silu", need_input_grad=need_in), nn.Linear(h, h, act="silu"),
                         nn.Linear(h, o, out_fp32=True))


def categorical_kl(lp, lq):
    """KL[p ‖ q] summed over groups for log-probabilities ``[..., G, C]``."""
    return (lp.exp() * (lp - lq)).sum((-1, -2))


class DreamerV3Agent:
    def __init__(self, cfg: DreamerV3Config = None, n_envs: int = 8, device="cpu"):
        self.cfg = c = cfg or DreamerV3Config()
        self.device, self.n_envs = torch.device(device), n_envs
        nn.manual_seed(c.seed)
        Z, D, H, A = c.groups * c.classes, c.deter, c.hidden, c.act_dim
        self.Z = Z
        dev = self.device
        self.enc = _mlp(c.obs_dim, H, H, need_in=False).to(dev)
        self.inp = nn.Linear(Z + A, H, act="silu").to(dev)
        self.gru = nn.GRUCell(H, D).to(dev)
        self.prior = _mlp(D, H, Z).to(dev)
        self.post = _mlp(D + H, H, Z).to(dev)
        self.dec = _mlp(D + Z, H, c.obs_dim).to(dev)
        self.rew = _mlp(D + Z, H, c.bins).to(dev)
        self.cont = _mlp(D + Z, H, 1).to(dev)
        self.actor = _mlp(D + Z, H, 2 * A).to(dev)
        self.critic = _mlp(D + Z, H, c.bins).to(dev)
        self.critic_slow = _mlp(D + Z, H, c.bins).to(dev)
        self.critic_slow.copy_from(self.critic)
        wm = [("enc.", self.enc), ("inp.", self.inp), ("gru.", self.gru), ("prior.", self.prior), ("post.", self.post),
              ("dec.", self.dec), ("rew.", self.rew), ("cont.", self.cont)]
        self.wm_opt = nn.Adam([np for pre, m in wm for np in m.named_params(pre)], lr=c.lr)
        self.actor_opt = nn.Adam(self.actor.named_params("actor."), lr=c.ac_lr)
        self.critic_opt = nn.Adam(self.critic.named_params("critic."), lr=c.ac_lr)
        for o in (self.wm_opt, self.actor_opt, self.critic_opt):
            o.max_grad_norm = c.max_grad_norm
        self.binv = torch.linspace(-c.bin_range, c.bin_range, c.bins, device=dev)
        self.gen = torch.Generator(device=dev).manual_seed(c.seed + 1)
        W, E = c.window, n_envs
        z = dict(device=dev)
        self.obs_buf = torch.zeros(W, E, c.obs_dim, **z)
        self.act_buf = torch.zeros(W, E, A, **z)           # action taken AFTER seeing obs_buf[t]
        self.rew_buf = torch.zeros(W, E, **z)              # reward received on arriving at obs_buf[t]
        self.first_buf = torch.zeros(W, E, **z)            # obs_buf[t] starts an episode
        self.term_buf = torch.zeros(W, E, **z)             # obs_buf[t] is terminal
        self.pos = torch.zeros(E, dtype=torch.long, device=dev)      # rows written per env (each env has its own stream)
        self.ret_range = 1.0
        self._h = torch.zeros(E, c.deter, **z)
        self._z = torch.zeros(E, Z, **z)
        self._a = torch.zeros(E, A, **z)
        self.last: Dict[str, float] = {}

    # ------------------------------------------------------------------ pieces
    def _x(self, t):
        return t.to(torch.bfloat16) if self.device.type == "cuda" else t.float()

    def _logp(self, logits):
        """Log-probabilities ``[..., G, C]`` with the uniform mix."""
        c = self.cfg
        p = torch.softmax(logits.float().reshape(*logits.shape[:-1], c.groups, c.classes), -1)
        return torch.log((1 - c.unimix) * p + c.unimix / c.classes)

    def _sample(self, logp):
        """One-hot sample with straight-through gradient, flattened to ``[..., G·C]``."""
        p = logp.exp()
        idx = torch.multinomial(p.reshape(-1, self.cfg.classes), 1, generator=self.gen)[:, 0]
        hot = F.one_hot(idx, self.cfg.classes).to(p.dtype).reshape(p.shape)
        return (hot + p - p.detach()).reshape(*p.shape[:-2], self.Z)

    def _step(self, h, z, a, call):
        """h' = GRU(inp([z, a]), h).  ``call(module, *xs)`` is ``nn.apply`` in training and a plain forward when acting."""
        x = call(self.inp, self._x(torch.cat([z, a], -1)))
        return call(self.gru, self._x(x), self._x(h)).float()

    @staticmethod
    def _fwd(module, *xs):
        return module.forward(*xs)

    def actor_dist(self, feat, call):
        out = call(self.actor, self._x(feat)).float()
        A = self.cfg.act_dim
        mean, std = torch.tanh(out[:, :A]), 0.1 + 0.9 * torch.sigmoid(out[:, A:] + 2.0)
        return mean, std

    # ------------------------------------------------------------------ acting (filtering with the posterior)
    @torch.no_grad()
    def select_action(self, obs, first=None, explore=True):
        c = self.cfg
        if first is not None:
            keep = (1 - first.float())[:, None]
            self._h, self._z, self._a = self._h * keep, self._z * keep, self._a * keep
        h = self._step(self._h, self._z, self._a, self._fwd)
        e = self.enc.forward(self._x(symlog(obs.float()))).float()
        z = self._sample(self._logp(self.post.forward(self._x(torch.cat([h, e], -1))))).detach()
        mean, std = self.actor_dist(torch.cat([h, z], -1), self._fwd)
        a = mean + std * torch.randn(mean.shape, device=self.device, generator=self.gen) if explore else mean
        a = a.clamp(-1, 1)
        self._h, self._z, self._a = h, z, a
        return a

    def record(self, obs, action, reward, first, terminal, mask=None):
        """Append one row to the stream of every env (or of the envs in ``mask``)."""
        e = torch.arange(self.n_envs, device=self.device) if mask is None else mask.nonzero(as_tuple=False)[:, 0]
        i = self.pos[e] % self.cfg.window
        self.obs_buf[i, e], self.act_buf[i, e], self.rew_buf[i, e] = obs[e], action[e], reward[e]
        self.first_buf[i, e], self.term_buf[i, e] = first[e], terminal[e]
        self.pos[e] += 1

    @property
    def t(self):
        return int(self.pos.min())

    # ------------------------------------------------------------------ world model
    def _observe(self, obs, act, first):
        """Posterior filtering over a batch of sequences ``[T, B, ·]`` inside the autograd graph."""
        c, (T, B) = self.cfg, obs.shape[:2]
        h = torch.zeros(B, c.deter, device=self.device)
        z = torch.zeros(B, self.Z, device=self.device)
        a = torch.zeros(B, c.act_dim, device=self.device)
        hs, zs, lps, lqs = [], [], [], []
        for t in range(T):
            keep = (1 - first[t])[:, None]
            h, z, a = h * keep, z * keep, a * keep
            h = self._step(h, z, a, nn.apply)
            e = nn.apply(self.enc, self._x(symlog(obs[t]))).float()
            lq = self._logp(nn.apply(self.post, self._x(torch.cat([h, e], -1))))
            lp = self._logp(nn.apply(self.prior, self._x(h)))
            z = self._sample(lq)
            hs.append(h), zs.append(z), lps.append(lp), lqs.append(lq)
            a = act[t]
        return torch.stack(hs), torch.stack(zs), torch.stack(lps), torch.stack(lqs)

    def _batch(self):
        c, W = self.cfg, self.cfg.window
        T, B = c.seq_len, c.batch
        e = torch.randint(0, self.n_envs, (B,), device=self.device, generator=self.gen)
        end = self.pos[e]
        lo = (end - W).clamp(min=0)
        span = (end - T + 1 - lo).clamp(min=1)
        t0 = lo + (torch.rand(B, device=self.device, generator=self.gen) * span).long().clamp(max=span - 1)
        idx = (t0[None] + torch.arange(T, device=self.device)[:, None]) % W                     # [T, B]
        first = self.first_buf[idx, e[None]].clone()
        first[0] = 1.0                                                                           # no state is carried in
        return self.obs_buf[idx, e[None]], self.act_buf[idx, e[None]], self.rew_buf[idx, e[None]], first, self.term_buf[idx, e[None]]

    def train_world_model(self, batch):
        c = self.cfg
        obs, act, rew, first, term = batch
        T, B = obs.shape[:2]
        hs, zs, lp, lq = self._observe(obs, act, first)
        feat = torch.cat([hs, zs], -1).reshape(T * B, -1)
        rec = nn.apply(self.dec, self._x(feat)).float()
        rl = nn.apply(self.rew, self._x(feat)).float()
        cl = nn.apply(self.cont, self._x(feat)).float()[:, 0]
        loss_rec = (rec - symlog(obs.reshape(T * B, -1))).pow(2).sum(-1).mean()
        valid_r = (1 - first.reshape(-1))                                                        # no reward on a first step
        loss_rew = (-(two_hot(symlog(rew.reshape(-1)), self.binv) * torch.log_softmax(rl, -1)).sum(-1) * valid_r).sum() / valid_r.sum().clamp(min=1)
        loss_cont = F.binary_cross_entropy_with_logits(cl, 1 - term.reshape(-1))
        kl_dyn = categorical_kl(lq.detach(), lp).clamp(min=c.free_bits).mean()
        kl_rep = categorical_kl(lq, lp.detach()).clamp(min=c.free_bits).mean()
        loss = loss_rec + loss_rew + loss_cont + c.beta_dyn * kl_dyn + c.beta_rep * kl_rep
        loss.backward()
        if c.max_grad_norm > 0:
            self.wm_opt.clip()
        self.wm_opt.step(zero_grad=True)
        out = dict(recon=loss_rec, reward_loss=loss_rew, cont_loss=loss_cont, kl=categorical_kl(lq, lp).mean())
        return hs.detach().reshape(T * B, -1), zs.detach().reshape(T * B, -1), (1 - term.reshape(-1)), {k: float(v.detach()) for k, v in out.items()}

    # ------------------------------------------------------------------ behaviour
    def _value(self, net, feat, call):
        logits = call(net, self._x(feat)).float()
        return symexp((torch.softmax(logits, -1) * self.binv).sum(-1)), logits

    def imagine(self, h, z, call):
        """Roll the prior forward with actor actions.  Returns features ``[H+1, N, D+Z]``, actions, means / stds."""
        c = self.cfg
        feats, acts, ents = [torch.cat([h, z], -1)], [], []
        for _ in range(c.imag_horizon):
            mean, std = self.actor_dist(feats[-1].detach(), call)
            a = (mean + std * torch.randn(mean.shape, device=self.device, generator=self.gen)).clamp(-1, 1)
            h = self._step(h, z, a, call)
            z = self._sample(self._logp(call(self.prior, self._x(h))))
            feats.append(torch.cat([h, z], -1)), acts.append(a), ents.append(torch.log(std).sum(-1))
        return torch.stack(feats), torch.stack(acts), torch.stack(ents)

    def train_behaviour(self, h0, z0, cont0):
        c = self.cfg
        feats, acts, ents = self.imagine(h0, z0, nn.apply)                                       # gradient flows through the dynamics
        Hh, N = c.imag_horizon, h0.shape[0]
        flat = feats.reshape((Hh + 1) * N, -1)
        rew = symexp((torch.softmax(nn.apply(self.rew, self._x(flat)).float(), -1) * self.binv).sum(-1)).reshape(Hh + 1, N)
        cont = torch.sigmoid(nn.apply(self.cont, self._x(flat)).float()[:, 0]).reshape(Hh + 1, N)
        cont = torch.cat([cont0[None], cont[1:]], 0)
        with torch.no_grad():
            v_slow, _ = self._value(self.critic_slow, flat, self._fwd)
        v, _ = self._value(self.critic, flat, nn.apply)
        v = v.reshape(Hh + 1, N)
        disc = c.gamma * cont
        ret = [v[-1]]
        for t in range(Hh - 1, -1, -1):                                                          # λ-return, reward on arrival at t+1
            ret.append(rew[t + 1] + disc[t + 1] * ((1 - c.lam) * v[t + 1] + c.lam * ret[-1]))
        ret = torch.stack(ret[::-1][:-1])                                                        # [H, N]
        weight = torch.cumprod(torch.cat([cont0[None], disc[1:-1]], 0), 0).detach()          # nothing follows a terminal start
        lo, hi = torch.quantile(ret.detach().flatten(), 0.05), torch.quantile(ret.detach().flatten(), 0.95)
        self.ret_range = 0.99 * self.ret_range + 0.01 * float(hi - lo)
        actor_loss = -(weight * (ret / max(1.0, self.ret_range) + c.entropy_coef * ents)).mean()
        actor_loss.backward()
        if c.max_grad_norm > 0:
            self.actor_opt.clip()
        self.actor_opt.step(zero_grad=True)
        self.wm_opt.arena.grd.zero_()                       # dynamics / heads only carried the gradient to the actor
        self.critic_opt.arena.grd.zero_()
        # critic: two-hot regression onto the λ-returns plus a pull towards its own slow copy
        fd = feats[:-1].detach().reshape(Hh * N, -1)
        logits = nn.apply(self.critic, self._x(fd)).float()
        tgt = two_hot(symlog(ret.detach().reshape(-1)), self.binv)
        with torch.no_grad():
            slow = torch.softmax(self.critic_slow.forward(self._x(fd)).float(), -1)
        logp = torch.log_softmax(logits, -1)
        critic_loss = (weight.reshape(-1) * (-(tgt * logp).sum(-1) - c.critic_reg * (slow * logp).sum(-1))).mean()
        critic_loss.backward()
        if c.max_grad_norm > 0:
            self.critic_opt.clip()
        self.critic_opt.step(zero_grad=True)
        self.critic_slow.polyak_from(self.critic, 1 - c.critic_ema)
        return dict(actor_loss=float(actor_loss.detach()), critic_loss=float(critic_loss.detach()), imag_return=float(ret.detach().mean()),
                    imag_value_slow=float(v_slow.mean()))

    def train_step(self):
        if min(self.t, self.cfg.window) < self.cfg.seq_len:
            return None
        h, z, cont, out = self.train_world_model(self._batch())
        out.update(self.train_behaviour(h, z, cont))
        self.last = out
        return out

    def save(self, path):
        from ..io.checkpoint import save_checkpoint
        mods = dict(enc=self.enc, inp=self.inp, gru=self.gru, prior=self.prior, post=self.post, dec=self.dec, rew=self.rew,
                    cont=self.cont, actor=self.actor, critic=self.critic)
        save_checkpoint(path, [np for k, m in mods.items() for np in m.named_params(k + ".")], [], {"steps": float(self.t)})


def run_dreamerv3(env, agent: DreamerV3Agent, total_env_steps: int, seed_steps: int = 500, train_every: int = 2):
    """Act with the filtered posterior state, record ``(obs, action, reward-on-arrival, first, terminal)`` rows, train every
    ``train_every`` env batches after ``seed_steps``.  Returns finished episode returns."""
    dev, c = agent.device, agent.cfg
    obs = env.reset_batch().float().clone()
    first = torch.ones(env.n_envs, device=dev)
    rew_in = torch.zeros(env.n_envs, device=dev)
    ep_ret = torch.zeros(env.n_envs, device=dev)
    finished, step, it = [], 0, 0
    while step < total_env_steps:
        a = agent.select_action(obs, first=first, explore=True)
        if step < seed_steps:
            a = torch.rand(env.n_envs, c.act_dim, device=dev) * 2 - 1
            agent._a = a
        agent.record(obs, a, rew_in, first, torch.zeros_like(first))
        nxt, r, done, term = env.step_batch(a)
        r, done, term = r.float(), done.float(), term.float()
        ep_ret += r
        if bool(done.any()):
            # the last observation of an episode gets its own row (reward on arrival, terminal flag) in the streams of
            # the envs that ended, before their reset observation
            agent.record(env.next_obs.float(), torch.zeros_like(a), r, torch.zeros_like(first), term, mask=done.bool())
            finished.extend(ep_ret[done.bool()].tolist())
            ep_ret[done.bool()] = 0
        obs, first, rew_in = nxt.float().clone(), done.clone(), r * (1 - done)
        step += env.n_envs
        it += 1
        if step >= seed_steps and it % train_every == 0:
            agent.train_step()
    return finished
