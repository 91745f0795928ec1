"""Imitation from demonstrations: behaviour cloning, demonstration collection, and demo-seeded off-policy RL.

``collect_demos``   roll a policy (a scripted controller, a trained agent, a tele-operator callback) in a batched env and
                    write the transitions to the trajectory container (``data.datasets.TrajectoryWriter``), one episode
                    per env stream
``BCTrainer``       regress actions on observations from a demonstration set: MSE, or the negative log-likelihood of a
                    Gaussian head with a learned state-independent log-σ; observation normalisation from the demo
                    statistics; minibatch epochs on the device-resident set (``training.Trainer`` underneath for MSE)
``HilSerlTrainer``  SAC whose every batch is half demonstrations, half online data (a pinned demo prefix of the replay,
                    ``StoreReplay.mixed_indices``), with human interventions: a transition whose action was overridden
                    by the operator is stored in the online part AND appended to the demonstrations
(noeira/deep_agents/bc/, noeira/deep_agents/demos/, noeira/deep_agents/hil_serl/.)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional

import numpy as np
import torch

from .. import nn
from ..data.replay import StoreReplay
from .sac import SACConfig, SACTrainer


# ------------------------------------------------------------------------------------------ demonstrations
def collect_demos(env, policy: Callable, n_episodes: int, path: Optional[str] = None, max_steps: int = 10_000) -> Dict[str, np.ndarray]:
    """Runs ``policy(obs) → action`` until ``n_episodes`` episodes finished.  Returns the flat transition arrays (and writes
    one container episode per finished env episode when ``path`` is given)."""
    from ..data.datasets import TrajectoryWriter
    E = env.n_envs
    obs = env.reset_batch().float().clone()
    cur = [dict(obs=[], action=[], reward=[], next_obs=[], done=[]) for _ in range(E)]
    done_eps = []
    for _ in range(max_steps):
        a = policy(obs).float()
        nxt, r, done, term = env.step_batch(a)
        true_next = env.next_obs.float() if hasattr(env, "next_obs") else nxt.float()
        for e in range(E):
            c = cur[e]
            c["obs"].append(obs[e].cpu().numpy()), c["action"].append(a[e].cpu().numpy()), c["reward"].append([float(r[e])])
            c["next_obs"].append(true_next[e].cpu().numpy()), c["done"].append([float(term[e])])
            if bool(done[e]):
                done_eps.append({k: np.asarray(v, np.float32) for k, v in c.items()})
                cur[e] = dict(obs=[], action=[], reward=[], next_obs=[], done=[])
        obs = nxt.float().clone()
        if len(done_eps) >= n_episodes:
            break
    done_eps = done_eps[:n_episodes]
    if path is not None and done_eps:
        fields = {k: v.shape[1] for k, v in done_eps[0].items()}
        w = TrajectoryWriter(path, fields, meta={"episodes": len(done_eps)})
        for ep in done_eps:
            w.add_episode(**ep)
        w.close()
    return {k: np.concatenate([ep[k] for ep in done_eps]) for k in done_eps[0]} if done_eps else {}


def load_demos(path: str) -> Dict[str, np.ndarray]:
    from ..data.datasets import TrajectoryStore
    return TrajectoryStore(path).all_steps()


# ------------------------------------------------------------------------------------------ behaviour cloning
@dataclass
class BCConfig:
    obs_dim: int = 3
    act_dim: int = 1
    hidden: int = 128
    lr: float = 1e-3
    batch: int = 256
    loss: str = "mse"                 # "mse" | "nll"
    normalize_obs: bool = True
    action_scale: float = 1.0
    seed: int = 0


class BCTrainer:
    def __init__(self, cfg: BCConfig, obs, act, device="cpu"):
        self.cfg, self.device = cfg, torch.device(device)
        nn.manual_seed(cfg.seed)
        obs = torch.as_tensor(obs, dtype=torch.float32, device=self.device)
        act = torch.as_tensor(act, dtype=torch.float32, device=self.device)
        self.mean = obs.mean(0) if cfg.normalize_obs else torch.zeros(cfg.obs_dim, device=self.device)
        self.std = obs.std(0).clamp_min(1e-3) if cfg.normalize_obs else torch.ones(cfg.obs_dim, device=self.device)
        self.x, self.y = (obs - self.mean) / self.std, act / cfg.action_scale
        self.net = nn.Sequential(nn.LinearReLU(cfg.obs_dim, cfg.hidden, need_input_grad=False), nn.LinearReLU(cfg.hidden, cfg.hidden),
                                 nn.GaussianHead(cfg.hidden, cfg.act_dim, log_std_init=-1.0)).to(self.device)
        self.opt = nn.Adam(self.net.named_params(), lr=cfg.lr)
        self.gen = torch.Generator(device=self.device).manual_seed(cfg.seed + 1)

    def _in(self, x):
        return x.to(torch.bfloat16) if self.device.type == "cuda" else x

    def train_epoch(self) -> float:
        c, n = self.cfg, self.x.shape[0]
        perm = torch.randperm(n, device=self.device, generator=self.gen)
        head = self.net.mods[2]
        total, nb = 0.0, 0
        for b0 in range(0, n - c.batch + 1, c.batch) if n >= c.batch else [0]:
            idx = perm[b0: b0 + c.batch]
            xb, yb = self.x[idx], self.y[idx]
            mu = self.net.forward(self._in(xb)).float()
            if c.loss == "mse":
                loss, dmu = nn.losses.mse_per_sample(mu, yb)
                loss, dmu = loss.mean(), dmu / mu.shape[0]
            else:
                ls = head.log_std.data.float().expand_as(mu)
                loss, dmu, dls = nn.losses.gaussian_nll(mu, ls, yb, head.LS_MIN, head.LS_MAX)
                head.log_std.grad.add_(dls.sum(0))
            self.net.vjp(dmu if self.device.type == "cpu" else dmu.to(torch.bfloat16))
            self.opt.step(zero_grad=True)
            total, nb = total + float(loss), nb + 1
        return total / max(nb, 1)

    @torch.no_grad()
    def act(self, obs):
        x = (obs.to(self.device).float() - self.mean) / self.std
        return (self.net.forward(self._in(x)).float() * self.cfg.action_scale).clamp(-self.cfg.action_scale, self.cfg.action_scale)

    def save(self, path):
        from ..io.checkpoint import save_checkpoint
        save_checkpoint(path, list(self.net.named_params()), [], {})


# ------------------------------------------------------------------------------------------ demo-seeded SAC with interventions
class HilSerlTrainer:
    def __init__(self, cfg: SACConfig, demos: Dict[str, np.ndarray], capacity: int = 100_000, device="cpu", demo_fraction: float = 0.5,
                 demo_capacity: Optional[int] = None):
        self.cfg, self.device, self.demo_fraction = cfg, torch.device(device), demo_fraction
        self.sac = SACTrainer(cfg, device)
        n = demos["obs"].shape[0]
        self.demo_cap = demo_capacity or 2 * n
        self.replay = StoreReplay(self.demo_cap + capacity, cfg.obs_dim, cfg.act_dim, device=self.device, demo_prefix=self.demo_cap,
                                  seed=cfg.seed)
        t = lambda k: torch.as_tensor(demos[k], dtype=torch.float32, device=self.device)
        self.n_demo = 0
        self._add_demo(t("obs"), t("action"), t("reward").reshape(-1), t("next_obs"), t("done").reshape(-1))
        self.interventions = 0

    def _add_demo(self, s, a, r, sp, d):
        k = min(s.shape[0], self.demo_cap - self.n_demo)
        i = slice(self.n_demo, self.n_demo + k)
        rp = self.replay
        rp.s[i], rp.a[i], rp.r[i], rp.sp[i], rp.d[i] = s[:k], a[:k], r[:k], sp[:k], d[:k]
        self.n_demo += k

    def select_action(self, obs, deterministic=False):
        return self.sac.select_action(obs, deterministic)

    def store(self, s, a, r, sp, d, intervened=None):
        """Online transitions; rows with ``intervened`` (the operator's action was executed) also join the demonstrations."""
        self.replay.store_batch(s, a, r, sp, d)
        if intervened is not None and bool(intervened.any()):
            m = intervened.bool()
            self._add_demo(s[m], a[m], r[m], sp[m], d[m])
            self.interventions += int(m.sum())

    def update(self):
        rp, B = self.replay, self.cfg.batch
        nd = int(B * self.demo_fraction)
        di = torch.randint(0, max(self.n_demo, 1), (nd,), device=self.device, generator=rp.gen)
        online = max(rp.size - rp.base, 0)
        oi = rp.base + torch.randint(0, max(online, 1), (B - nd,), device=self.device, generator=rp.gen) if online > 0 else \
            torch.randint(0, max(self.n_demo, 1), (B - nd,), device=self.device, generator=rp.gen)
        return self.sac.update(*rp.gather(torch.cat([di, oi])))
