"""Classic-control environments, batched as tensor programs (run on CPU or CUDA tensors alike):
``PendulumEnv`` (swing-up, continuous torque), ``CartPoleEnv`` (continuous force variant of the discrete task),
``MountainCarContinuousEnv``.  Same ``BatchedEnv`` surface as the physics environments: ``reset_batch``,
``step_batch(action) -> (obs, reward, done, terminated)`` with automatic per-lane reset and ``next_obs`` holding the
pre-reset observation.  Dynamics constants follow the Gymnasium definitions the reference's native versions use
(noeira/envs/pendulum, cartpole, mountain_car; "145x faster than Gymnasium" native CartPole).
"""
from __future__ import annotations

import math

import torch

from .batched_env import BatchedEnv


class _TensorEnv(BatchedEnv):
    obs_dim = act_dim = 0
    max_steps = 200
    graph_safe = False           # steps are tensor operations drawing from the environment's own generator

    def __init__(self, n_envs: int, device="cpu", seed: int = 0):
        self.n_envs, self.device = int(n_envs), torch.device(device)
        self.gen = torch.Generator(device=self.device).manual_seed(seed)
        z = dict(device=self.device, dtype=torch.float32)
        self.obs = torch.zeros(n_envs, self.obs_dim, **z)
        self.next_obs = torch.zeros(n_envs, self.obs_dim, **z)
        self.reward = torch.zeros(n_envs, **z)
        self.done = torch.zeros(n_envs, **z)
        self.terminated = torch.zeros(n_envs, **z)
        self.steps = torch.zeros(n_envs, device=self.device, dtype=torch.int32)
        self.ep_return = torch.zeros(n_envs, **z)
        self.finished_return = torch.zeros(n_envs, **z)
        self.ep_stats = torch.zeros(4, **z)        # Σ finished returns, finished episodes, Σ rewards, steps
        self.state = None

    # ---- the engine-style surface the on-policy trainers drive (PPO steps ``env.engine`` into its own rollout buffers)
    @property
    def engine(self):
        return self

    @property
    def obs_pad(self) -> int:
        return (self.obs_dim + 63) // 64 * 64

    @property
    def obs_bf16(self) -> torch.Tensor:
        buf = torch.zeros(self.n_envs, self.obs_pad, device=self.device, dtype=torch.bfloat16)
        buf[:, : self.obs_dim].copy_(self.obs)
        return buf

    def step(self, action, reward, done, terminated, obs_f32=None, obs_bf16=None, next_obs_f32=None, next_obs_bf16=None,
             finished_return=None, do_reset=True, ep_stats=None, dbg=None):
        self.step_batch(action, auto_reset=do_reset)
        reward.copy_(self.reward), done.copy_(self.done), terminated.copy_(self.terminated)
        for dst, src in ((obs_f32, self.obs), (obs_bf16, self.obs), (next_obs_f32, self.next_obs), (next_obs_bf16, self.next_obs)):
            if dst is not None and dst is not src:
                dst[:, : self.obs_dim].copy_(src)
        if finished_return is not None and finished_return is not self.finished_return:
            finished_return.copy_(self.finished_return)

    def _rand(self, *shape):
        return torch.rand(*shape, device=self.device, generator=self.gen)

    def _sample_state(self, n):
        raise NotImplementedError

    def _observe(self, s):
        raise NotImplementedError

    def _dynamics(self, s, a):
        """→ (next state, reward, terminated)"""
        raise NotImplementedError

    def reset_batch(self):
        self.state = self._sample_state(self.n_envs)
        self.steps.zero_()
        self.ep_return.zero_()
        self.obs.copy_(self._observe(self.state))
        return self.obs

    def step_batch(self, action, auto_reset: bool = True):
        a = action.to(self.device, torch.float32).reshape(self.n_envs, -1)[:, : self.act_dim]   # padded action rows are fine
        s2, r, term = self._dynamics(self.state, a)
        self.steps += 1
        trunc = self.steps >= self.max_steps
        done = term | trunc
        self.reward.copy_(r)
        self.terminated.copy_(term.float())
        self.done.copy_(done.float())
        self.ep_return += r
        self.next_obs.copy_(self._observe(s2))
        self.pre_reset_state = s2
        self.ep_stats[2] += r.sum()
        self.ep_stats[3] += self.n_envs
        if auto_reset:                                       # masked, without a host read: the step can sit in a captured stream
            fin = done.to(r.dtype)
            self.finished_return.copy_(torch.where(done, self.ep_return, self.finished_return))
            self.ep_stats[0] += (self.ep_return * fin).sum()
            self.ep_stats[1] += fin.sum()
            fresh = self._sample_state(self.n_envs)
            s2 = torch.where(done.reshape(-1, *([1] * (s2.dim() - 1))), fresh, s2)
            self.steps.masked_fill_(done, 0)
            self.ep_return.masked_fill_(done, 0.0)
        self.state = s2
        self.obs.copy_(self._observe(s2))
        return self.obs, self.reward, self.done, self.terminated


class PendulumEnv(_TensorEnv):
    obs_dim, act_dim, max_steps = 3, 1, 200
    max_speed, max_torque, dt, g, m, l = 8.0, 2.0, 0.05, 10.0, 1.0, 1.0

    def _sample_state(self, n):
        return torch.stack([(self._rand(n) * 2 - 1) * math.pi, (self._rand(n) * 2 - 1)], 1)

    def _observe(self, s):
        return torch.stack([torch.cos(s[:, 0]), torch.sin(s[:, 0]), s[:, 1]], 1)

    def _dynamics(self, s, a):
        th, thd = s[:, 0], s[:, 1]
        u = a[:, 0].clamp(-1, 1) * self.max_torque
        ang = ((th + math.pi) % (2 * math.pi)) - math.pi
        cost = ang ** 2 + 0.1 * thd ** 2 + 0.001 * u ** 2
        thd2 = (thd + (3 * self.g / (2 * self.l) * torch.sin(th) + 3.0 / (self.m * self.l ** 2) * u) * self.dt).clamp(-self.max_speed, self.max_speed)
        return torch.stack([th + thd2 * self.dt, thd2], 1), -cost, torch.zeros_like(th, dtype=torch.bool)


class CartPoleEnv(_TensorEnv):
    obs_dim, act_dim, max_steps = 4, 1, 500
    gravity, mc, mp, length, force_mag, tau = 9.8, 1.0, 0.1, 0.5, 10.0, 0.02

    def _sample_state(self, n):
        return (self._rand(n, 4) - 0.5) * 0.1

    def _observe(self, s):
        return s

    def _dynamics(self, s, a):
        x, xd, th, thd = s.unbind(1)
        f = a[:, 0].clamp(-1, 1) * self.force_mag
        ct, st = torch.cos(th), torch.sin(th)
        total, pml = self.mc + self.mp, self.mp * self.length
        tmp = (f + pml * thd ** 2 * st) / total
        thacc = (self.gravity * st - ct * tmp) / (self.length * (4.0 / 3.0 - self.mp * ct ** 2 / total))
        xacc = tmp - pml * thacc * ct / total
        s2 = torch.stack([x + self.tau * xd, xd + self.tau * xacc, th + self.tau * thd, thd + self.tau * thacc], 1)
        term = (s2[:, 0].abs() > 2.4) | (s2[:, 2].abs() > 12 * math.pi / 180)
        return s2, torch.ones_like(x), term


class MountainCarContinuousEnv(_TensorEnv):
    obs_dim, act_dim, max_steps = 2, 1, 999
    power, goal = 0.0015, 0.45

    def _sample_state(self, n):
        return torch.stack([self._rand(n) * 0.2 - 0.6, torch.zeros(n, device=self.device)], 1)

    def _observe(self, s):
        return s

    def _dynamics(self, s, a):
        p, v = s[:, 0], s[:, 1]
        f = a[:, 0].clamp(-1, 1)
        v2 = (v + f * self.power - 0.0025 * torch.cos(3 * p)).clamp(-0.07, 0.07)
        p2 = (p + v2).clamp(-1.2, 0.6)
        v2 = torch.where((p2 <= -1.2) & (v2 < 0), torch.zeros_like(v2), v2)
        term = p2 >= self.goal
        return torch.stack([p2, v2], 1), term.float() * 100.0 - 0.1 * f ** 2, term


class AcrobotEnv(_TensorEnv):
    """Two-link underactuated pendulum (torque on the second joint only), the book dynamics integrated with one RK4 step of
    0.2 s; reward −1 per step until the tip is above the bar by one link length.  Action in [−1, 1] scales the torque."""
    obs_dim, act_dim, max_steps = 6, 1, 500
    m1 = m2 = 1.0
    l1 = 1.0
    lc1 = lc2 = 0.5
    i1 = i2 = 1.0
    g, dt = 9.8, 0.2

    def _sample_state(self, n):
        return (self._rand(n, 4) - 0.5) * 0.2

    def _observe(self, s):
        return torch.stack([torch.cos(s[:, 0]), torch.sin(s[:, 0]), torch.cos(s[:, 1]), torch.sin(s[:, 1]), s[:, 2], s[:, 3]], 1)

    def _deriv(self, s, u):
        t1, t2, d1, d2 = s.unbind(1)
        m1, m2, l1, lc1, lc2, i1, i2, g = self.m1, self.m2, self.l1, self.lc1, self.lc2, self.i1, self.i2, self.g
        dd1 = m1 * lc1 ** 2 + m2 * (l1 ** 2 + lc2 ** 2 + 2 * l1 * lc2 * torch.cos(t2)) + i1 + i2
        dd2 = m2 * (lc2 ** 2 + l1 * lc2 * torch.cos(t2)) + i2
        phi2 = m2 * lc2 * g * torch.cos(t1 + t2 - math.pi / 2)
        phi1 = -m2 * l1 * lc2 * d2 ** 2 * torch.sin(t2) - 2 * m2 * l1 * lc2 * d2 * d1 * torch.sin(t2) + \
            (m1 * lc1 + m2 * l1) * g * torch.cos(t1 - math.pi / 2) + phi2
        a2 = (u + dd2 / dd1 * phi1 - m2 * l1 * lc2 * d1 ** 2 * torch.sin(t2) - phi2) / (m2 * lc2 ** 2 + i2 - dd2 ** 2 / dd1)
        a1 = -(dd2 * a2 + phi1) / dd1
        return torch.stack([d1, d2, a1, a2], 1)

    def _dynamics(self, s, a):
        u = a[:, 0].clamp(-1, 1)
        k1 = self._deriv(s, u)
        k2 = self._deriv(s + 0.5 * self.dt * k1, u)
        k3 = self._deriv(s + 0.5 * self.dt * k2, u)
        k4 = self._deriv(s + self.dt * k3, u)
        s2 = s + self.dt / 6 * (k1 + 2 * k2 + 2 * k3 + k4)
        wrap = lambda x: ((x + math.pi) % (2 * math.pi)) - math.pi
        s2 = torch.stack([wrap(s2[:, 0]), wrap(s2[:, 1]), s2[:, 2].clamp(-4 * math.pi, 4 * math.pi), s2[:, 3].clamp(-9 * math.pi, 9 * math.pi)], 1)
        term = (-torch.cos(s2[:, 0]) - torch.cos(s2[:, 0] + s2[:, 1])) > 1.0
        return s2, torch.where(term, torch.zeros_like(u), -torch.ones_like(u)), term


class DiscreteActions:
    """A batched env with continuous actions driven by a table of discrete ones: action index i → ``table[i]``
    (two pushes for CartPole, three torques for Acrobot or MountainCar)."""

    def __init__(self, env, table):
        self.env = env
        self.table = torch.as_tensor(table, dtype=torch.float32, device=env.device).reshape(len(table), -1)
        self.n_actions = self.table.shape[0]

    def __getattr__(self, k):
        return getattr(self.env, k)

    def reset_batch(self):
        return self.env.reset_batch()

    def step_batch(self, a, auto_reset: bool = True):
        return self.env.step_batch(self.table[a.long().reshape(-1)], auto_reset=auto_reset)

    def selective_reset_batch(self):
        pass
