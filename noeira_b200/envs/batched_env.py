"""Batched environment API: every env of the batch lives on the device, and the trainer only
enqueues kernels (reference surface: ``BatchedEnv`` — noeira/deep_agents/training/batched_env.mojo:80-142,
``GPUContinuousEnv`` static kernels — noeira/core/env_traits.mojo:599-810).

Contract
    reset_batch()                      re-initialise every env, fills ``obs``
    step_batch(action)                 consumes ``action [N, act_dim]`` and fills
                                       ``obs`` (post-reset), ``next_obs`` (pre-reset, the bootstrap state),
                                       ``reward``, ``done`` (terminated | truncated), ``terminated``
    selective_reset_batch()            resets the envs whose ``done`` flag is set (the physics envs fuse
                                       this into ``step_batch`` and make it a no-op)
All outputs are persistent tensors (fixed addresses), so a step can be captured in a CUDA graph.
``obs_bf16`` is a zero-padded bf16 mirror with a 16-byte aligned row stride, written by the same
kernel, so the policy GEMM can TMA-load it without a cast pass.
"""
from __future__ import annotations

import torch


def _pad_to(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class BatchedEnv:
    n_envs: int
    obs_dim: int
    act_dim: int

    def _alloc_io(self, device):
        z = dict(device=device, dtype=torch.float32)
        self.obs = torch.zeros(self.n_envs, self.obs_dim, **z)
        self.next_obs = torch.zeros(self.n_envs, self.obs_dim, **z)
        self.obs_pad = _pad_to(self.obs_dim, 64)
        self.obs_bf16 = torch.zeros(self.n_envs, self.obs_pad, device=device, dtype=torch.bfloat16)
        self.next_obs_bf16 = torch.zeros(self.n_envs, self.obs_pad, device=device, dtype=torch.bfloat16)
        self.reward = torch.zeros(self.n_envs, **z)
        self.done = torch.zeros(self.n_envs, **z)
        self.terminated = torch.zeros(self.n_envs, **z)
        self.finished_return = torch.full((self.n_envs,), float("nan"), **z)
        # device accumulators: Σ finished returns, finished episodes, Σ reward, Σ finished episode lengths
        self.ep_stats = torch.zeros(4, **z)

    def reset_batch(self):
        raise NotImplementedError

    def step_batch(self, action):
        raise NotImplementedError

    def selective_reset_batch(self):
        pass


class Physics3dBatchedEnv(BatchedEnv):
    """Batched physics env over the fused step kernel
    (reference: ``Phyics3dBatchedEnv`` — noeira/envs/phyics3d_batched_env.mojo:120, step_batch :1260-1516)."""

    def __init__(self, model, n_envs: int, task=None, device="cuda", seed: int = 0):
        from ..physics.engine import PhysicsEngine, TaskSpec
        self.engine = PhysicsEngine(model, n_envs, task or TaskSpec(), device=device, seed=seed)
        self.n_envs = int(n_envs)
        self.obs_dim = self.engine.nobs
        self.act_dim = model.nu
        self.device = self.engine.device
        self._alloc_io(self.device)

    def reset_batch(self):
        self.engine.reset(self.obs, self.obs_bf16)
        return self.obs

    def step_batch(self, action, dbg=None, auto_reset: bool = True):
        """``auto_reset=False`` keeps finished lanes where they are (planning rollouts, evaluation of fixed horizons)."""
        self.engine.step(action, self.reward, self.done, self.terminated, obs_f32=self.obs, obs_bf16=self.obs_bf16,
                         next_obs_f32=self.next_obs, next_obs_bf16=self.next_obs_bf16,
                         finished_return=self.finished_return, do_reset=auto_reset, ep_stats=self.ep_stats, dbg=dbg)
        return self.obs, self.reward, self.done, self.terminated


class PlanarChainEnv(Physics3dBatchedEnv):
    """7-capsule planar chain: obs 17 = qpos[1:] ‖ qvel, act 6, reward = forward velocity − 0.1‖a‖²,
    dt 0.01 × 5 substeps, PGS 8 iterations, friction 0.4."""

    def __init__(self, n_envs: int, device="cuda", seed: int = 0, model_seed: int = 0, max_steps: int = 1000):
        from ..physics.engine import TaskSpec
        from ..physics.model import planar_chain
        super().__init__(planar_chain(seed=model_seed), n_envs,
                         TaskSpec(frame_skip=5, max_steps=max_steps, forward_dof=0, w_forward=1.0, w_ctrl=0.1),
                         device=device, seed=seed)


class HalfCheetahEnv(Physics3dBatchedEnv):
    """HalfCheetah-class runner (noeira/envs/half_cheetah/half_cheetah_config.mojo:23-96)."""

    def __init__(self, n_envs: int, device="cuda", seed: int = 0, max_steps: int = 1000):
        from ..physics.engine import TaskSpec
        from ..physics.model import half_cheetah
        super().__init__(half_cheetah(), n_envs, TaskSpec(frame_skip=5, max_steps=max_steps), device=device, seed=seed)


class HopperEnv(Physics3dBatchedEnv):
    def __init__(self, n_envs: int, device="cuda", seed: int = 0, max_steps: int = 1000):
        from ..physics.engine import TaskSpec
        from ..physics.model import hopper
        super().__init__(hopper(), n_envs,
                         TaskSpec(frame_skip=4, max_steps=max_steps, w_ctrl=1e-3, w_alive=1.0, term_dof=1,
                                  term_lo=-0.55, term_hi=1e30, reset_noise_pos=5e-3, reset_noise_vel=5e-3),
                         device=device, seed=seed)


class Walker2dEnv(Physics3dBatchedEnv):
    """Walker2d-class biped: reward = forward velocity + alive bonus − 1e-3 ‖a‖², ends when the torso drops below 0.8 m
    (root z coordinate relative to its start) or after ``max_steps``."""

    def __init__(self, n_envs: int, device="cuda", seed: int = 0, max_steps: int = 1000):
        from ..physics.engine import TaskSpec
        from ..physics.model import walker2d
        super().__init__(walker2d(), n_envs,
                         TaskSpec(frame_skip=4, max_steps=max_steps, w_ctrl=1e-3, w_alive=1.0, term_dof=1, term_lo=-0.45, term_hi=0.75,
                                  reset_noise_pos=5e-3, reset_noise_vel=5e-3), device=device, seed=seed)


class InvertedDoublePendulumEnv(Physics3dBatchedEnv):
    """Balance two poles in series on a cart: alive bonus while the first pole stays within ±0.35 rad of upright."""

    def __init__(self, n_envs: int, device="cuda", seed: int = 0, max_steps: int = 1000):
        from ..physics.engine import TaskSpec
        from ..physics.model import inverted_double_pendulum
        super().__init__(inverted_double_pendulum(), n_envs,
                         TaskSpec(frame_skip=5, max_steps=max_steps, w_forward=0.0, w_ctrl=1e-3, w_alive=10.0, term_dof=1, term_lo=-0.35,
                                  term_hi=0.35, obs_qpos_skip=0, reset_noise_pos=0.05, reset_noise_vel=0.05), device=device, seed=seed)


class InvertedPendulumEnv(Physics3dBatchedEnv):
    """Balance one pole on a cart: alive bonus while the pole stays within ±0.2 rad."""

    def __init__(self, n_envs: int, device="cuda", seed: int = 0, max_steps: int = 1000):
        from ..physics.engine import TaskSpec
        from ..physics.model import pendulum_cart
        super().__init__(pendulum_cart(), n_envs,
                         TaskSpec(frame_skip=2, max_steps=max_steps, w_forward=0.0, w_ctrl=0.0, w_alive=1.0, term_dof=1, term_lo=-0.2,
                                  term_hi=0.2, obs_qpos_skip=0, reset_noise_pos=0.01, reset_noise_vel=0.01), device=device, seed=seed)


class ReacherEnv(Physics3dBatchedEnv):
    """Two-link arm in the plane; the built-in task rewards small controls while the policy moves joint 0 forward (the
    target-reaching reward of the original needs a per-env goal: use the task layer's goal predicates for that)."""

    def __init__(self, n_envs: int, device="cuda", seed: int = 0, max_steps: int = 50):
        from ..physics.engine import TaskSpec
        from ..physics.model import reacher
        super().__init__(reacher(), n_envs, TaskSpec(frame_skip=2, max_steps=max_steps, w_forward=1.0, w_ctrl=0.1, obs_qpos_skip=0),
                         device=device, seed=seed)
