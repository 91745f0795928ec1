"""Shared RL training infrastructure: running statistics, episode bookkeeping, cadence, and the two generic batched
drivers that every agent goes through.

  RunningMeanStd       CleanRL-style running mean / variance with the parallel (Welford) batch merge, tensor based so the
                       same object runs on CPU or on the device without a host round trip; ``skip`` rows are left out;
                       ``save`` / ``load`` use the reference's three-line text format (``count`` / ``mean`` / ``var``).
                       (noeira/deep_agents/training/obs_norm.mojo:32-126, device twins :158-260)
  norm_reward          ``r / sqrt(var(discounted return) + 1e-8)`` clipped (obs_norm.mojo:128-137)
  EpisodeTracker       rolling window over recent episode returns, pre-filled with a baseline
                       (noeira/deep_agents/training/episode_tracker.mojo:16-64)
  EpisodeReturnRing    device ring of finished-episode returns, read back every ``sync_every`` iterations only
  DeviceMeanAccum      Σ / count pairs kept on the device, read on demand (device_mean_accum.mojo:157)
  Cadence              "every N env steps" trigger that survives steps of any stride (print / eval / checkpoint)
  run_onpolicy_train_batched / run_offpolicy_train_batched
                       the loops of noeira/deep_agents/training/driver_onpolicy.mojo:479 and driver_offpolicy.mojo:823:
                       act → step_batch → record → (train) → selective reset, with print / checkpoint / logger cadence
                       and the episode window; the env and the agent stay on one device and exchange tensors.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, field
from typing import Callable, List, Optional

import torch


class RunningMeanStd:
    def __init__(self, dim: int, device="cpu", dtype=torch.float64):
        self.dim = int(dim)
        self.mean = torch.zeros(dim, device=device, dtype=dtype)
        self.var = torch.ones(dim, device=device, dtype=dtype)
        self.count = torch.full((1,), 1e-4, device=device, dtype=dtype)

    def update(self, x: torch.Tensor, skip: Optional[torch.Tensor] = None):
        """Merge a batch ``x [N, dim]``; rows with ``skip`` set (diverged lanes) are left out.  No host sync."""
        x = x.reshape(-1, self.dim).to(self.mean.dtype)
        if skip is not None:
            keep = (~skip.reshape(-1).bool()).to(x.dtype)
            n = keep.sum()
            safe = n.clamp_min(1.0)
            bm = (x * keep[:, None]).sum(0) / safe
            bv = (((x - bm) ** 2) * keep[:, None]).sum(0) / safe
        else:
            n = torch.tensor(float(x.shape[0]), device=x.device, dtype=x.dtype)
            bm = x.mean(0)
            bv = x.var(0, unbiased=False)
        tot = self.count + n
        delta = bm - self.mean
        m2 = self.var * self.count + bv * n + delta * delta * self.count * n / tot
        live = (n > 0).to(x.dtype)                               # an all-skipped batch changes nothing
        self.mean += live * delta * n / tot
        self.var.copy_(live * (m2 / tot) + (1 - live) * self.var)
        self.count.copy_(live * tot + (1 - live) * self.count)

    def normalize(self, x: torch.Tensor, clip: float = 10.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        y = ((x.to(self.mean.dtype) - self.mean) / torch.sqrt(self.var + 1e-8)).clamp(-clip, clip)
        if out is not None:
            out.copy_(y)
            return out
        return y.to(x.dtype)

    def save(self, path: str):
        lines = ["count " + repr(float(self.count)), "mean " + " ".join(repr(float(v)) for v in self.mean.cpu()),
                 "var " + " ".join(repr(float(v)) for v in self.var.cpu())]
        tmp = path + ".tmp"
        with open(tmp, "w") as f:
            f.write("\n".join(lines) + "\n")
        os.replace(tmp, path)

    def load(self, path: str):
        rows = [ln.split(" ") for ln in open(path).read().split("\n") if ln]
        self.count.fill_(float(rows[0][1]))
        self.mean.copy_(torch.tensor([float(v) for v in rows[1][1: 1 + self.dim]], dtype=self.mean.dtype))
        self.var.copy_(torch.tensor([float(v) for v in rows[2][1: 1 + self.dim]], dtype=self.var.dtype))


def norm_reward(r: torch.Tensor, ret_var: torch.Tensor, clip: float = 10.0) -> torch.Tensor:
    """CleanRL ``NormalizeReward``: reward over the standard deviation of the discounted return, clipped."""
    return (r / torch.sqrt(ret_var.to(r.dtype) + 1e-8)).clamp(-clip, clip)


class ReturnNormalizer:
    """Discounted-return tracker feeding ``norm_reward``: ``ret = ret·γ·(1−done) + r``; its running variance scales
    the rewards (one per lane, device resident)."""

    def __init__(self, n_envs: int, gamma: float, device="cpu", clip: float = 10.0):
        self.gamma, self.clip = gamma, clip
        self.ret = torch.zeros(n_envs, device=device, dtype=torch.float64)
        self.rms = RunningMeanStd(1, device=device)

    def __call__(self, reward: torch.Tensor, done: torch.Tensor) -> torch.Tensor:
        self.ret.mul_(self.gamma).add_(reward.to(self.ret.dtype))
        self.rms.update(self.ret[:, None])
        out = norm_reward(reward, self.rms.var[0], self.clip)
        self.ret.mul_(1.0 - done.to(self.ret.dtype))
        return out


class EpisodeTracker:
    def __init__(self, window_size: int = 100, initial_fill: float = 0.0):
        self.window = [float(initial_fill)] * window_size
        self.window_size, self.idx, self.current_return, self.ep_count = window_size, 0, 0.0, 0

    def add_reward(self, reward: float):
        self.current_return += float(reward)

    def end_episode(self):
        self.add_complete_return(self.current_return)
        self.current_return = 0.0

    def add_complete_return(self, ret: float):
        self.window[self.idx] = float(ret)
        self.idx = (self.idx + 1) % self.window_size
        self.ep_count += 1

    def mean_return(self) -> float:
        return sum(self.window) / self.window_size


class EpisodeReturnRing:
    """Finished-episode returns collected ON the device; the host reads the ring every ``sync_every`` pushes only (the
    reference's deferred episode readback of the device rollout, ``episode_sync_every``)."""

    def __init__(self, capacity: int, device="cpu", sync_every: int = 32):
        self.buf = torch.zeros(capacity + 1, device=device)              # last slot: where lanes that are not done write
        self.head = torch.zeros(1, dtype=torch.int64, device=device)      # total returns ever written
        self.capacity, self.sync_every, self._pushes, self._read = capacity, sync_every, 0, 0

    def push(self, finished_return: torch.Tensor, done: torch.Tensor):
        """``finished_return [N]`` is valid where ``done [N]`` is set.  Pure tensor ops (capturable, no host sync)."""
        d = done.reshape(-1) > 0.5
        rank = torch.cumsum(d.to(torch.int64), 0) - 1
        pos = torch.where(d, (self.head + rank) % self.capacity, torch.full_like(rank, self.capacity))
        self.buf.index_copy_(0, pos, finished_return.reshape(-1).to(self.buf.dtype))
        self.head += d.sum()
        self._pushes += 1

    def due(self) -> bool:
        return self._pushes % self.sync_every == 0

    def drain(self, tracker: EpisodeTracker) -> int:
        """Read back what was finished since the last drain (one host sync) into the tracker."""
        head = int(self.head.item())
        n = min(head - self._read, self.capacity)
        if n > 0:
            idx = torch.arange(head - n, head, device=self.buf.device) % self.capacity
            for r in self.buf[idx].cpu().tolist():
                tracker.add_complete_return(r)
        self._read = head
        return max(n, 0)


class DeviceMeanAccum:
    """Named Σ / count pairs on the device: ``add`` is a tensor op, ``read`` the only host sync."""

    def __init__(self, names: List[str], device="cpu"):
        self.names = list(names)
        self.acc = torch.zeros(len(names), 2, device=device, dtype=torch.float64)

    def add(self, name: str, value: torch.Tensor, count: float = 1.0):
        i = self.names.index(name)
        self.acc[i, 0] += value.reshape(()).to(self.acc.dtype) if torch.is_tensor(value) else float(value)
        self.acc[i, 1] += count

    def read(self, reset: bool = True):
        a = self.acc.cpu()
        out = {n: (float(a[i, 0] / a[i, 1]) if a[i, 1] > 0 else float("nan")) for i, n in enumerate(self.names)}
        if reset:
            self.acc.zero_()
        return out


class Cadence:
    """True once for every multiple of ``every`` that ``step`` passes, whatever the stride of the steps."""

    def __init__(self, every: int):
        self.every, self._next = int(every), int(every)

    def __call__(self, step: int) -> bool:
        if self.every <= 0 or step < self._next:
            return False
        self._next = (step // self.every + 1) * self.every
        return True


@dataclass
class TrainLog:
    steps: List[int] = field(default_factory=list)
    mean_returns: List[float] = field(default_factory=list)
    episodes: int = 0


def _episode_bookkeeping(env, ring: EpisodeReturnRing, tracker: EpisodeTracker, force: bool = False):
    ring.push(env.finished_return, env.done)
    if force or ring.due():
        ring.drain(tracker)


def run_onpolicy_train_batched(trainer, env, total_env_steps: int, *, print_every: int = 0, logger=None,
                               checkpoint_every: int = 0, checkpoint_path: str = "", episode_sync_every: int = 32,
                               window_size: int = 100, initial_fill: float = 0.0, base_step: int = 0,
                               on_iteration: Optional[Callable] = None, verbose: bool = False,
                               read_metrics_every: int = 1) -> TrainLog:
    """Generic on-policy loop.  ``trainer`` provides either the device rollout (``train_iteration`` +
    ``env_steps_per_iteration``: PPO on the device, episode statistics come from ``env.ep_stats``) or the step-wise
    interface ``select_action_batched(obs) → action``, ``record_batch(obs, action, reward, next_obs, done, terminated)``
    and ``train_step() → metrics | None`` (fires at the rollout boundary).  Returns the logged window means."""
    log = TrainLog()
    tracker = EpisodeTracker(window_size, initial_fill)
    ring = EpisodeReturnRing(max(4 * env.n_envs, 1024), device=env.obs.device, sync_every=episode_sync_every)
    pr, ck = Cadence(print_every), Cadence(checkpoint_every)
    step = base_step
    device_rollout = hasattr(trainer, "train_iteration")
    if not device_rollout:
        env.reset_batch()
    last = {}
    it = 0
    while step - base_step < total_env_steps:
        it += 1
        if device_rollout:
            # metrics live on the device; reading them is the only host sync of an iteration
            m = trainer.train_iteration(read_metrics=(it % max(read_metrics_every, 1) == 0))
            step += trainer.env_steps_per_iteration
            if m and m.get("episodes", 0) > 0:
                for _ in range(int(min(m["episodes"], window_size))):
                    tracker.add_complete_return(m["mean_episode_return"])
        else:
            obs = env.obs.clone()
            action = trainer.select_action_batched(obs)
            env.step_batch(action)
            trainer.record_batch(obs, action, env.reward, env.next_obs, env.done, env.terminated)
            _episode_bookkeeping(env, ring, tracker)
            env.selective_reset_batch()
            step += env.n_envs
            m = trainer.train_step()
        if m:
            last = m
            if on_iteration is not None:
                on_iteration(step, m)
        if pr(step - base_step) or step - base_step >= total_env_steps:
            if not device_rollout:
                ring.drain(tracker)
            log.steps.append(step)
            log.mean_returns.append(tracker.mean_return())
            log.episodes = tracker.ep_count
            if logger is not None:
                logger.log_scalars(step, dict(last, mean_return=tracker.mean_return(), episodes=tracker.ep_count))
            if verbose:
                print(f"[on-policy] step {step}  episodes {tracker.ep_count}  mean return {tracker.mean_return():.2f}")
        if checkpoint_path and ck(step - base_step):
            trainer.save(checkpoint_path)
    if checkpoint_path:
        trainer.save(checkpoint_path)
    return log


def run_offpolicy_train_batched(agent, env, replay, total_env_steps: int, *, learning_starts: int = 1000, utd: int = 1,
                                batch_size: int = 256, print_every: int = 0, logger=None, checkpoint_every: int = 0,
                                checkpoint_path: str = "", eval_every: int = 0, eval_fn: Optional[Callable] = None,
                                episode_sync_every: int = 32, window_size: int = 100, initial_fill: float = 0.0,
                                base_step: int = 0, verbose: bool = False) -> TrainLog:
    """Generic off-policy loop (SAC / TD3 / DDPG / DQN-style agents): uniform-random actions until ``learning_starts``,
    then per env step: act → ``step_batch`` → store to the replay → ``utd`` updates → selective reset; print / eval /
    checkpoint cadences.  ``agent``: ``select_action(obs)``, ``update(s, a, r, sp, d)`` (or ``update_captured``),
    ``save(path)``; ``replay``: ``store_batch`` and ``sample(batch) → ((s, a, r, sp, d), idx, w)``."""
    log = TrainLog()
    tracker = EpisodeTracker(window_size, initial_fill)
    ring = EpisodeReturnRing(max(4 * env.n_envs, 1024), device=env.obs.device, sync_every=episode_sync_every)
    pr, ck, ev = Cadence(print_every), Cadence(checkpoint_every), Cadence(eval_every)
    dev = env.obs.device
    obs = env.reset_batch().clone()
    step = base_step
    pad = (env.act_dim + 7) // 8 * 8
    act_buf = torch.zeros(env.n_envs, pad, device=dev)
    update = getattr(agent, "update_captured", None) or agent.update
    metrics = {}
    while step - base_step < total_env_steps:
        if step - base_step < learning_starts:
            a = torch.rand(env.n_envs, env.act_dim, device=dev) * 2 - 1
        else:
            a = agent.select_action(obs).float()
        act_buf[:, : env.act_dim] = a
        env.step_batch(act_buf)
        replay.store_batch(obs, a, env.reward, env.next_obs, env.terminated)
        _episode_bookkeeping(env, ring, tracker)
        env.selective_reset_batch()
        obs = env.obs.clone()
        step += env.n_envs
        if step - base_step >= learning_starts:
            for _ in range(utd):
                res = replay.sample(batch_size)
                batch = res[0] if isinstance(res[0], (tuple, list)) else res      # device stores also return indices / weights
                metrics = update(*batch) or metrics
        if pr(step - base_step) or step - base_step >= total_env_steps:
            ring.drain(tracker)
            log.steps.append(step)
            log.mean_returns.append(tracker.mean_return())
            log.episodes = tracker.ep_count
            if logger is not None and metrics:      # rows start with the first update: every row then has the same columns
                row = {k: float(v) for k, v in metrics.items()}
                logger.log_scalars(step, dict(row, mean_return=tracker.mean_return(), episodes=tracker.ep_count))
            if verbose:
                print(f"[off-policy] step {step}  episodes {tracker.ep_count}  mean return {tracker.mean_return():.2f}")
        if eval_fn is not None and ev(step - base_step):
            eval_fn(step)
        if checkpoint_path and ck(step - base_step):
            agent.save(checkpoint_path)
    if checkpoint_path and hasattr(agent, "save"):
        agent.save(checkpoint_path)
    return log
