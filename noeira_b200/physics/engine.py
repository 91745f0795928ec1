"""Device side of the physics engine: state tensors + launch of the fused step kernel.

State layout per env (`torch` tensors on the GPU, AoS so one warp reads one env contiguously):
``qpos [N, nv]``, ``qvel [N, nv]``, ``warm [N, nlimit + 3·ncs]`` (constraint multipliers kept per
fixed slot for warm starting), ``step_count [N]`` int32, ``ep_return [N]``.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np
import torch

from .._native import check, cuda_lib, ptr, stream_ptr
from .model import RigidModel

PHYS_WARPS = 8


class PhysParams(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in (
        "nbody", "nv", "nvp", "nlimit", "ncs", "nu", "maxdepth", "rmax",
        "imodel_words", "fmodel_words", "warp_words", "warm_words",
        "frame_skip", "pgs_iters", "friction_rows", "max_steps",
        "forward_dof", "term_dof", "obs_qpos_skip", "pad0")] + [(n, ctypes.c_float) for n in (
        "dt", "gx", "gy", "gz",
        "solref_tc", "solref_dr", "solimp_d0", "solimp_dmax", "solimp_width", "solimp_mid", "solimp_pow", "margin",
        "plane_nx", "plane_ny", "plane_nz", "plane_off",
        "friction_reg", "max_vel", "obs_clip", "pad1",
        "w_forward", "w_ctrl", "w_alive", "term_lo", "term_hi", "pad2", "pad3", "pad4")]


@dataclass
class TaskSpec:
    """Reward / termination of a locomotion-style task built on the engine."""
    frame_skip: int = 5
    max_steps: int = 1000
    forward_dof: int = 0
    w_forward: float = 1.0
    w_ctrl: float = 0.1
    w_alive: float = 0.0
    term_dof: int = -1
    term_lo: float = -1e30
    term_hi: float = 1e30
    obs_qpos_skip: int = 1
    obs_clip: float = 100.0
    reset_noise_pos: float = 0.1
    reset_noise_vel: float = 0.1


def make_params(m: RigidModel, task: TaskSpec) -> PhysParams:
    o = m.opt
    P = PhysParams()
    P.nbody, P.nv, P.nlimit, P.ncs, P.nu, P.maxdepth, P.rmax = m.nbody, m.nv, m.nlimit, m.ncs, m.nu, m.maxdepth, o.rmax
    P.nvp = m.nv | 1
    i32, f32 = m.pack((task.reset_noise_pos, task.reset_noise_vel))
    P.imodel_words = (len(i32) + 3) // 4 * 4
    P.fmodel_words = (len(f32) + 3) // 4 * 4
    nb, nv, nvp, rmax = m.nbody, m.nv, P.nvp, o.rmax
    P.warm_words = (m.nlimit + 3 * m.ncs + 3) // 4 * 4
    # persistent arrays + the larger of (packed Delassus triangle, the per-body arrays it overlays); see `carve`
    scratch = nb * 3 + nb * 9 + nv * 6 + nv * nvp + 128 + 2 * rmax * nvp + rmax * 8 + max(32 * 33 // 2, nb * (4 + 10 * 2 + 6 * 2))
    P.warp_words = (scratch + 3) // 4 * 4 + P.warm_words
    P.frame_skip, P.pgs_iters, P.max_steps = task.frame_skip, o.pgs_iters, task.max_steps
    P.friction_rows = 0 if not o.friction_rows else (1 if m.planar else 2)
    P.forward_dof, P.term_dof, P.obs_qpos_skip = task.forward_dof, task.term_dof, task.obs_qpos_skip
    P.dt = o.timestep
    P.gx, P.gy, P.gz = o.gravity
    P.solref_tc, P.solref_dr = o.solref
    P.solimp_d0, P.solimp_dmax, P.solimp_width, P.solimp_mid, P.solimp_pow = o.solimp
    P.margin = o.margin
    P.plane_nx, P.plane_ny, P.plane_nz = o.plane_normal
    P.plane_off = o.plane_offset
    P.friction_reg, P.max_vel, P.obs_clip = o.friction_reg, o.max_vel, task.obs_clip
    P.w_forward, P.w_ctrl, P.w_alive, P.term_lo, P.term_hi = task.w_forward, task.w_ctrl, task.w_alive, task.term_lo, task.term_hi
    return P


class PhysicsEngine:
    """Batched simulator: N envs of one model on one GPU."""

    def __init__(self, model: RigidModel, n_envs: int, task: TaskSpec = None, device="cuda", seed: int = 0):
        self.model = model
        self.task = task or TaskSpec()
        self.n = int(n_envs)
        self.device = torch.device(device)
        self.P = make_params(model, self.task)
        i32, f32 = model.pack((self.task.reset_noise_pos, self.task.reset_noise_vel))
        i32 = np.pad(i32, (0, self.P.imodel_words - len(i32)))
        f32 = np.pad(f32, (0, self.P.fmodel_words - len(f32)))
        self.imodel = torch.from_numpy(i32).to(self.device)
        self.fmodel = torch.from_numpy(f32).to(self.device)
        nv = model.nv
        self.nwarm = model.nlimit + 3 * model.ncs
        z = dict(device=self.device, dtype=torch.float32)
        self.qpos = torch.zeros(self.n, nv, **z)
        self.qvel = torch.zeros(self.n, nv, **z)
        self.warm = torch.zeros(self.n, max(self.nwarm, 1), **z)
        self.step_count = torch.zeros(self.n, device=self.device, dtype=torch.int32)
        self.ep_return = torch.zeros(self.n, **z)
        self.rng_counter = torch.zeros(1, device=self.device, dtype=torch.int64)
        self.seed = int(seed)
        self.nobs = (nv - self.task.obs_qpos_skip) + nv
        self._lib = cuda_lib()
        self._reset_count = 0

    # ------------------------------------------------------------------ kernels
    def reset(self, obs_f32=None, obs_bf16=None, mask=None):
        self._reset_count += 1
        st = obs_bf16.stride(0) if obs_bf16 is not None else 0
        check(self._lib.nb_phys_env_reset(
            ctypes.byref(self.P), ptr(self.fmodel), ptr(self.qpos), ptr(self.qvel), ptr(self.warm),
            ptr(self.step_count), ptr(self.ep_return), ptr(mask), ptr(obs_f32), ptr(obs_bf16), ctypes.c_int(st),
            ctypes.c_ulonglong(self.seed), ctypes.c_ulonglong(self._reset_count << 32), ctypes.c_int(self.n),
            stream_ptr()), "phys_env_reset")

    def step(self, action, reward, done, terminated, obs_f32=None, obs_bf16=None, next_obs_f32=None,
             next_obs_bf16=None, finished_return=None, do_reset=True, ep_stats=None, dbg=None):
        """One control step for every env. `action` is [N, >=nu] fp32 (row stride taken from the tensor)."""
        st = 0
        for t in (obs_bf16, next_obs_bf16):
            if t is not None:
                st = t.stride(0)
        check(self._lib.nb_phys_env_step(
            ctypes.byref(self.P), ptr(self.imodel), ptr(self.fmodel), ptr(self.qpos), ptr(self.qvel), ptr(self.warm),
            ptr(self.step_count), ptr(self.ep_return), ptr(action), ctypes.c_int(action.stride(0)),
            ptr(obs_f32), ptr(obs_bf16), ctypes.c_int(st), ptr(next_obs_f32), ptr(next_obs_bf16),
            ptr(reward), ptr(done), ptr(terminated), ptr(finished_return), ptr(self.rng_counter),
            ctypes.c_ulonglong(self.seed), ctypes.c_int(self.n), ctypes.c_int(1 if do_reset else 0), ptr(ep_stats), ptr(dbg),
            stream_ptr()), "phys_env_step")
        # device resident counter → fresh reset noise on every (captured) replay
        self.rng_counter.add_(1)

    def body_poses(self):
        xpos = torch.empty(self.n, self.model.nbody, 3, device=self.device)
        xmat = torch.empty(self.n, self.model.nbody, 9, device=self.device)
        check(self._lib.nb_phys_fk(ctypes.byref(self.P), ptr(self.imodel), ptr(self.fmodel), ptr(self.qpos),
                                   ptr(xpos), ptr(xmat), ctypes.c_int(self.n), stream_ptr()), "phys_fk")
        return xpos, xmat
