"""LunarLander (continuous actions) as a batched environment over the 2-D rigid-body core.

On CUDA the step is one kernel (``csrc/lunar_lander.cu``: one thread per environment, step + reward + selective
reset); on the CPU the SAME source runs through the host library (``csrc/host/physics2d_host.cpp``), which is also the
oracle of the GPU test.  Lander hull and two legs on revolute joints (limits + spring-like motors), random height-field
terrain with a flat helipad, engines as impulses with dispersion noise, Gymnasium observation (8), shaping reward and
termination rules (crash / out of view −100, at rest +100).
Reference: noeira/envs/lunar_lander/lunar_lander.mojo, noeira/physics2d/.
"""
from __future__ import annotations

import ctypes

import torch

from .batched_env import BatchedEnv


class LunarLanderEnv(BatchedEnv):
    obs_dim, act_dim = 8, 2
    _name = "lunar"                # entry points nb_<name>_* (CUDA library) and nbh_<name>_* (host library)

    def __init__(self, n_envs: int, device="cuda", seed: int = 0):
        self.n_envs, self.device, self.seed = int(n_envs), torch.device(device), int(seed)
        self.on_cuda = self.device.type == "cuda"
        if self.on_cuda:
            from .._native import cuda_lib
            self.lib = cuda_lib()
            nbytes = int(self._fn("state_bytes")())
        else:
            from .._native import host_lib
            self.lib = host_lib()
            nbytes = int(self._fn("state_bytes")())
        self.state = torch.zeros(self.n_envs, nbytes, dtype=torch.uint8, device=self.device)
        self._alloc_io(self.device)
        self.engine = self            # the PPO device rollout drives an environment through ``env.engine.step``

    def _fn(self, what):
        return getattr(self.lib, f"{'nb' if self.on_cuda else 'nbh'}_{self._name}_{what}")

    def reset_batch(self):
        from .._native import check, ptr, stream_ptr
        if self.on_cuda:
            check(self._fn("reset")(ptr(self.state), ctypes.c_int(self.n_envs), ctypes.c_uint(self.seed), ptr(self.obs),
                                          ptr(self.obs_bf16), ctypes.c_int(self.obs_pad), stream_ptr()), f"{self._name}_reset")
        else:
            self._fn("reset")(ptr(self.state), ctypes.c_int(self.n_envs), ctypes.c_uint(self.seed), ptr(self.obs))
            self.obs_bf16[:, : self.obs_dim].copy_(self.obs)
        return self.obs

    def step(self, action, reward, done, terminated, obs_f32=None, obs_bf16=None, next_obs_f32=None, next_obs_bf16=None,
             finished_return=None, do_reset=True, ep_stats=None, dbg=None):
        """Engine-style step into caller-owned buffers (what a captured rollout uses)."""
        from .._native import check, ptr, stream_ptr
        assert action.dtype == torch.float32 and action.stride(-1) == 1
        c = ctypes
        if self.on_cuda:
            check(self._fn("step")(ptr(self.state), c.c_int(self.n_envs), c.c_uint(self.seed), ptr(action),
                                         c.c_int(action.stride(0)), ptr(reward), ptr(done), ptr(terminated), ptr(obs_f32),
                                         ptr(obs_bf16), ptr(next_obs_f32), ptr(next_obs_bf16),
                                         c.c_int((obs_bf16 if obs_bf16 is not None else self.obs_bf16).stride(0)),
                                         ptr(finished_return), ptr(ep_stats), c.c_int(1 if do_reset else 0), stream_ptr()),
                  f"{self._name}_step")
            return
        obs = obs_f32 if obs_f32 is not None else torch.empty_like(self.obs)
        nxt = next_obs_f32 if next_obs_f32 is not None else torch.empty_like(self.obs)
        fr = finished_return if finished_return is not None else torch.empty_like(self.reward)
        self._fn("step")(ptr(self.state), c.c_int(self.n_envs), c.c_uint(self.seed), ptr(action), c.c_int(action.stride(0)),
                                ptr(reward), ptr(done), ptr(terminated), ptr(obs), ptr(nxt), ptr(fr), c.c_int(1 if do_reset else 0))
        if obs_bf16 is not None:
            obs_bf16[:, : self.obs_dim].copy_(obs)
        if next_obs_bf16 is not None:
            next_obs_bf16[:, : self.obs_dim].copy_(nxt)
        if ep_stats is not None:
            fin = done > 0
            ep_stats[0] += torch.where(fin, fr, torch.zeros_like(fr)).sum()
            ep_stats[1] += fin.float().sum()
            ep_stats[2] += reward.sum()

    def step_batch(self, action, auto_reset: bool = True):
        a = action.to(self.device, torch.float32)
        a = a if a.stride(-1) == 1 else a.contiguous()
        self.step(a, self.reward, self.done, self.terminated, obs_f32=self.obs, obs_bf16=self.obs_bf16, next_obs_f32=self.next_obs,
                  next_obs_bf16=self.next_obs_bf16, finished_return=self.finished_return, do_reset=auto_reset,
                  ep_stats=self.ep_stats)
        return self.obs, self.reward, self.done, self.terminated

    def lander_pose(self) -> torch.Tensor:
        """[N, 6] x, y, angle, vx, vy, omega of the hull (state inspection in tests)."""
        return self.state.view(torch.float32)[:, :6].clone() if self.state.shape[1] % 4 == 0 else None


class BipedalWalkerEnv(LunarLanderEnv):
    """BipedalWalker: hull + two two-segment legs on motorised revolute joints, rolling random terrain, 10 lidar rays;
    observation (24), actions = four motor commands (sign = direction, magnitude = torque fraction), reward 130·Δx/30 minus
    posture and torque costs, −100 when the hull touches the ground.  Same structure as the lander: one CUDA thread per
    environment (``csrc/bipedal_walker.cu``), the same source on the host (``csrc/host/bipedal_host.cpp``).
    Reference: noeira/envs/bipedal_walker/."""
    obs_dim, act_dim = 24, 4
    _name = "bipedal"

    def hull_pose(self) -> torch.Tensor:
        return self.state.view(torch.float32)[:, :6].clone()

    lander_pose = hull_pose
