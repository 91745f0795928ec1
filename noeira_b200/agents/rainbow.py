"""Rainbow: the C51 learner with every extension switched on, each one a flag.

  distributional   categorical value distribution and projected Bellman target (``C51Trainer``)
  double Q         the online network picks the greedy next action, the target network evaluates it
  dueling          per-atom ``logit(s, a) = V(s) + A(s, a) − mean_a A(s, a)``
  noisy nets       ``nn.NoisyLinear`` in the hidden layer and both heads replaces ε-greedy exploration; the online network
                   draws fresh noise for every update and every acting call, the target network draws its own
  n-step returns   ``NStepCollector`` folds n consecutive transitions of every env of a batched env into one
  prioritised      proportional priorities = per-sample cross entropy, importance weights scale the loss

(noeira/deep_agents/c51/ holds the reference's Rainbow variant: noisy dueling C51 on a prioritised n-step replay.)
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import nn
from .discrete import C51Config, C51Trainer, _inp, project_distribution


@dataclass
class RainbowConfig(C51Config):
    noisy: bool = True
    dueling: bool = True
    n_step: int = 3
    prioritized: bool = True
    per_alpha: float = 0.5
    per_beta: float = 0.4
    sigma0: float = 0.5


class _DistHead(nn.Module):
    """Dueling head over atoms: value ``[B, 1, N]`` + advantage ``[B, A, N]`` − mean over actions."""

    def __init__(self, hidden, n_actions, n_atoms, noisy, sigma0):
        super().__init__()
        mk = (lambda i, o: nn.NoisyLinear(i, o, sigma0=sigma0, out_fp32=True)) if noisy else (lambda i, o: nn.Linear(i, o, out_fp32=True))
        self.v = self.add_child("value", mk(hidden, n_atoms))
        self.a = self.add_child("advantage", mk(hidden, n_actions * n_atoms))
        self.n_actions, self.n_atoms = n_actions, n_atoms

    def forward(self, h):
        B = h.shape[0]
        v = self.v.forward(h).float().reshape(B, 1, self.n_atoms)
        a = self.a.forward(h).float().reshape(B, self.n_actions, self.n_atoms)
        return (v + a - a.mean(1, keepdim=True)).reshape(B, -1)

    def vjp(self, dq):
        B = dq.shape[0]
        dq = dq.float().reshape(B, self.n_actions, self.n_atoms)
        dv = dq.sum(1)
        da = (dq - dq.mean(1, keepdim=True)).reshape(B, -1)
        return self.v.vjp(dv) + self.a.vjp(da)


def make_rainbow_network(cfg: RainbowConfig):
    hid = nn.Sequential(nn.NoisyLinear(cfg.hidden, cfg.hidden, sigma0=cfg.sigma0), nn.Elementwise("relu")) if cfg.noisy \
        else nn.LinearReLU(cfg.hidden, cfg.hidden)
    head = _DistHead(cfg.hidden, cfg.n_actions, cfg.n_atoms, cfg.noisy, cfg.sigma0) if cfg.dueling else (
        nn.NoisyLinear(cfg.hidden, cfg.n_actions * cfg.n_atoms, sigma0=cfg.sigma0, out_fp32=True) if cfg.noisy
        else nn.Linear(cfg.hidden, cfg.n_actions * cfg.n_atoms, out_fp32=True))
    return nn.Sequential(nn.LinearReLU(cfg.obs_dim, cfg.hidden, need_input_grad=False), hid, head)


class NStepCollector:
    """Turns the per-step transitions of a batched env into n-step transitions ``(s_t, a_t, Σ γ^k r_{t+k}, s_{t+m}, term, m)``
    where m ≤ n ends early at an episode end.  A ring of the last n steps per env lives on the device; ``push`` returns
    the transitions that became complete with this step."""

    def __init__(self, n: int, gamma: float, n_envs: int, obs_dim: int, device="cpu"):
        self.n, self.gamma, self.E = n, gamma, n_envs
        z = dict(device=device, dtype=torch.float32)
        self.s = torch.zeros(n, n_envs, obs_dim, **z)
        self.a = torch.zeros(n, n_envs, dtype=torch.long, device=device)
        self.r = torch.zeros(n, n_envs, **z)
        self.age = torch.zeros(n, n_envs, dtype=torch.long, device=device)      # rewards folded into the slot so far
        self.valid = torch.zeros(n, n_envs, dtype=torch.bool, device=device)
        self.head = 0

    def push(self, s, a, r, sp, terminated, done):
        """``sp`` is the true successor (before any reset), ``terminated`` stops bootstrapping, ``done`` ends the episode
        (termination or time limit).  Returns ``(s0, a0, R, sp, terminated, m)`` for every slot that reached n rewards
        or whose episode ended with this step.  The slot written now was emitted n − 1 pushes ago at the latest."""
        h = self.head
        self.s[h], self.a[h], self.r[h], self.age[h], self.valid[h] = s, a.long(), 0.0, 0, True
        self.r += torch.where(self.valid, (self.gamma ** self.age.float()) * r[None], torch.zeros_like(self.r))
        self.age += self.valid.long()
        emit = self.valid & ((self.age >= self.n) | done.bool()[None])
        idx = emit.nonzero(as_tuple=False)
        k, e = idx[:, 0], idx[:, 1]
        out = (self.s[k, e], self.a[k, e], self.r[k, e], sp[e], terminated[e].float(), self.age[k, e])
        self.valid &= ~emit
        self.head = (h + 1) % self.n
        return out


class RainbowTrainer(C51Trainer):
    def __init__(self, cfg: RainbowConfig = None, device="cpu"):
        cfg = cfg or RainbowConfig()
        super().__init__(cfg, device)
        nn.manual_seed(cfg.seed)
        self.q, self.q_target = make_rainbow_network(cfg).to(self.device), make_rainbow_network(cfg).to(self.device)
        self.q_target.copy_from(self.q)
        self.opt = nn.Adam(self.q.named_params(), lr=cfg.lr)
        self.opt.max_grad_norm = cfg.max_grad_norm

    def resample(self):
        if self.cfg.noisy:
            nn.reset_noise(self.q, self.gen)
            nn.reset_noise(self.q_target, self.gen)

    @torch.no_grad()
    def select_action(self, obs, explore=True):
        if not self.cfg.noisy:
            return super().select_action(obs, explore)
        self.q.train(explore)                       # acting greedily on the mean network when not exploring
        if explore:
            nn.reset_noise(self.q, self.gen)
            self.env_steps += obs.shape[0]
        a = self.q_values(obs).argmax(1)
        self.q.train(True)
        return a

    def update(self, s, a, r, sp, d, n_step=None, weights=None):
        """One gradient step.  ``n_step``: an int or a per-sample tensor of the number of rewards folded into ``r``
        (default: the configured n); ``weights``: importance weights of a prioritised draw.  Returns the loss and the
        per-sample cross entropies (the new priorities)."""
        c, B = self.cfg, s.shape[0]
        self.resample()
        ar = torch.arange(B, device=self.device)
        steps = c.n_step if n_step is None else n_step
        gam = c.gamma ** (steps.float() if torch.is_tensor(steps) else float(steps))
        with torch.no_grad():
            sel = self.q_values(sp).argmax(1)
            nxt = torch.softmax(self._dist(self.q_target, sp), -1)[ar, sel]
            if torch.is_tensor(gam):
                target = _project_per_sample(nxt, r.float(), d.float(), self.support, gam)
            else:
                target = project_distribution(nxt, r.float(), d.float(), self.support, gam)
        logits = self._dist(self.q, s)
        logp = torch.log_softmax(logits[ar, a.long()], -1)
        ce = -(target * logp).sum(-1)
        w = torch.ones(B, device=self.device) if weights is None else weights.float()
        loss = (w * ce).mean()
        dlog = torch.zeros_like(logits)
        dlog[ar, a.long()] = (logp.exp() - target) * (w / B)[:, None]
        self.q.vjp(dlog.reshape(B, -1))
        if c.max_grad_norm > 0:
            self.opt.clip()
        self.opt.step(zero_grad=True)
        self.updates += 1
        if self.updates % c.target_every == 0:
            self.q_target.copy_from(self.q)
        return dict(loss=loss, priorities=ce.detach(), mean_q=(logp.exp() * self.support).sum(-1).mean())


def _project_per_sample(next_probs, r, d, support, gamma_n):
    """``project_distribution`` with one discount per row."""
    B, N = next_probs.shape
    v_min, v_max = float(support[0]), float(support[-1])
    dz = (v_max - v_min) / (N - 1)
    tz = (r[:, None] + (gamma_n * (1 - d))[:, None] * support[None]).clamp(v_min, v_max)
    b = (tz - v_min) / dz
    lo, hi = b.floor().long(), b.ceil().long()
    same = (lo == hi).to(next_probs.dtype)
    out = torch.zeros_like(next_probs)
    out.scatter_add_(1, lo, next_probs * (hi.to(b.dtype) - b + same))
    out.scatter_add_(1, hi, next_probs * (b - lo.to(b.dtype)))
    return out


def run_rainbow(env, trainer: RainbowTrainer, total_steps: int, replay_capacity: int = 50000, learning_starts: int = 500,
                updates_per_step: int = 1, log=None):
    """Collect with the noisy (or ε-greedy) policy on a batched env with discrete actions, fold transitions into n-step
    ones, train from a proportional-priority replay.  Returns the list of finished-episode returns."""
    from ..data.replay import StoreReplay
    c, dev = trainer.cfg, trainer.device
    E = env.n_envs
    rep = StoreReplay(replay_capacity, c.obs_dim, 2, device=dev, seed=c.seed, per_alpha=c.per_alpha, per_beta=c.per_beta)
    nst = NStepCollector(c.n_step, c.gamma, E, c.obs_dim, device=dev)
    obs = env.reset_batch().float().clone()
    ep_ret = torch.zeros(E, device=dev)
    finished = []
    steps = 0
    while steps < total_steps:
        a = trainer.select_action(_inp(obs, dev))
        nxt, r, done, term = env.step_batch(a)               # ``nxt`` is already the reset observation where done
        true_next = env.next_obs.float() if hasattr(env, "next_obs") else nxt.float()
        r, done, term = r.float(), done.float(), term.float()
        s0, a0, R, sp, tm, k = nst.push(obs, a, r, true_next, term, done)
        if s0.shape[0]:
            rep.store_batch(s0, torch.stack([a0.float(), k.float()], 1), R, sp, tm)
        ep_ret += r
        if bool(done.any()):
            finished.extend(ep_ret[done.bool()].tolist())
            ep_ret[done.bool()] = 0
        obs = nxt.float().clone()
        steps += E
        if rep.size >= max(learning_starts, c.batch):
            for _ in range(updates_per_step):
                if c.prioritized:
                    idx, w = rep.per_indices(c.batch)
                else:
                    idx, w = rep.uniform_indices(c.batch), None
                s, ak, rr, spp, dd = rep.gather(idx)
                out = trainer.update(s, ak[:, 0].long(), rr, spp, dd, n_step=ak[:, 1], weights=w)
                if c.prioritized:
                    rep.update_priorities(idx, out["priorities"])
        if log is not None:
            log(steps, finished)
    return finished
