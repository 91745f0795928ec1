"""Top-down car racing as a batched environment: random closed tracks, a slip-based tire model on a rigid hull, tile-visit
reward, a 13-value state observation and an ego-centric grey-scale camera with frame stacking.

On CUDA the whole environment step is one kernel (``csrc/car_racing.cu::car_env_step_kernel``: one warp per lane of the
batch; the lanes of the warp share the track tiles, lane 0 integrates; reward, time limit, episode statistics, both
observations and the reset in the same launch) and the camera another (one CTA per lane of the batch culls the track to
the view, one thread per pixel).  The same arithmetic written with tensor operations (``_dynamics_tensor``,
``_render_tensor``) runs on CPU and is the oracle of the GPU tests.

Physics follows Gymnasium's ``car_dynamics.py`` constants on a single rigid hull, as the reference does
(noeira/physics2d/car/wheel_friction.mojo, car_dynamics.mojo, constants.mojo): per wheel the slip between the contact
patch and the ground gives a longitudinal and a lateral force proportional to slip, clipped to a friction circle that is
smaller on grass; the rear wheels are driven, all wheels brake, the front wheels steer through a rate-limited servo.
Environment rules follow noeira/envs/car_racing/car_racing.mojo (−0.1 per step, 1000 / tiles per newly visited tile, −100
outside the playfield, 1000 steps) and car_racing_pixel.mojo (grass 0.3 / road 0.7 / car 1.0, four stacked frames,
five discrete actions).  Tracks are periodic splines through twelve random check points, resampled to a fixed number of
tiles so that a whole batch shares one tensor layout.
"""
from __future__ import annotations

import ctypes
import math

import numpy as np
import torch

from .classic import DiscreteActions, _TensorEnv

SIZE = 0.02
HDR = 16          # x y angle vx vy omega | joint_fl joint_fr | wheel omega ×4 | track id | visited | gas | spare
SCALE = 6.0
PARAMS = dict(
    dt=1.0 / 50.0, engine_power=1e8 * SIZE * SIZE, brake_force=15.0, wheel_moment=4000 * SIZE * SIZE, wheel_radius=27 * SIZE,
    friction_limit=1e6 * SIZE * SIZE, friction_coef=205000 * SIZE * SIZE, grass_friction=0.6, steer_limit=0.4, steer_speed=3.0,
    steer_gain=50.0, hull_mass=10.0,
    # a 2.4 × 4.4 box of that mass; with explicit Euler the yaw damping of four tires (≈ 82 · Σ|r|² · dt / I per step) must
    # stay below 2, which an inertia of 10 does not give
    hull_inertia=10.0 * (2.4 ** 2 + 4.4 ** 2) / 12.0,
    half_width=40.0 / SCALE, playfield=2000.0 / SCALE, tile_reward=0.0, lap_fraction=0.95)
WHEEL_X = (-55 * SIZE, 55 * SIZE, -55 * SIZE, 55 * SIZE)        # front-left, front-right, rear-left, rear-right
WHEEL_Y = (80 * SIZE, 80 * SIZE, -82 * SIZE, -82 * SIZE)
CAR_HW, CAR_HL = 1.4, 2.8


def make_track(rng: np.random.Generator, tiles: int = 256, checkpoints: int = 12, radius: float = 900.0 / SCALE) -> np.ndarray:
    """A closed track [tiles, 2]: check points at jittered angles and random radii in [radius / 3, radius], a periodic
    Catmull–Rom spline through them, resampled at equal arc length; counter-clockwise, tile 0 is the start."""
    ang = (np.arange(checkpoints) + rng.uniform(0.0, 1.0, checkpoints) * 0.8) * 2 * math.pi / checkpoints
    rad = rng.uniform(radius / 3.0, radius, checkpoints)
    pts = np.stack([rad * np.cos(ang), rad * np.sin(ang)], 1)
    fine = []
    u = np.linspace(0.0, 1.0, 64, endpoint=False)[:, None]
    for i in range(checkpoints):
        p0, p1, p2, p3 = (pts[(i + k - 1) % checkpoints] for k in range(4))
        fine.append(0.5 * ((2 * p1) + (-p0 + p2) * u + (2 * p0 - 5 * p1 + 4 * p2 - p3) * u ** 2 + (-p0 + 3 * p1 - 3 * p2 + p3) * u ** 3))
    fine = np.concatenate(fine, 0)
    seg = np.linalg.norm(np.roll(fine, -1, 0) - fine, axis=1)
    arc = np.concatenate([[0.0], np.cumsum(seg)])
    want = np.linspace(0.0, arc[-1], tiles, endpoint=False)
    closed = np.concatenate([fine, fine[:1]], 0)
    return np.stack([np.interp(want, arc, closed[:, 0]), np.interp(want, arc, closed[:, 1])], 1).astype(np.float32)


def _seg_dist2(q, a, b):
    """Squared distance of points q [..., 1, 2] to segments a→b [T, 2] (broadcast) → [..., T]."""
    e, p = b - a, q - a
    l2 = (e * e).sum(-1)
    t = ((p * e).sum(-1) / l2.clamp_min(1e-12)).clamp(0.0, 1.0)
    d = p - t[..., None] * e
    return (d * d).sum(-1)


class CarRacingEnv(_TensorEnv):
    """Continuous actions (steer ∈ [−1, 1] with +1 = right, gas ∈ [0, 1], brake ∈ [0, 1]); observation = hull x, y, angle,
    vx, vy, yaw rate, the two steering angles, four wheel speeds, speed (13), optionally followed by ``lookahead`` track
    points ahead of the car in the car's frame (x right, y forward), which is what a state-based policy needs to drive."""
    act_dim, max_steps = 3, 1000

    def __init__(self, n_envs: int, device="cpu", seed: int = 0, n_tracks: int = 8, tiles: int = 256, lookahead: int = 0,
                 lookahead_stride: int = 4):
        self.tiles, self.lookahead, self.lookahead_stride = int(tiles), int(lookahead), int(lookahead_stride)
        self.obs_dim = 13 + 2 * self.lookahead
        super().__init__(n_envs, device, seed)
        rng = np.random.default_rng(seed)
        self.track = torch.from_numpy(np.stack([make_track(rng, tiles) for _ in range(n_tracks)])).to(self.device)
        self.params = dict(PARAMS, tile_reward=1000.0 / tiles)
        self._wx = torch.tensor(WHEEL_X, device=self.device)
        self._wy = torch.tensor(WHEEL_Y, device=self.device)
        self._cparams = (ctypes.c_float * 25)(*[float(v) for v in self.params.values()], *WHEEL_X, *WHEEL_Y)
        assert list(self.params) == list(PARAMS)
        self.use_kernels = self.device.type == "cuda"
        d = self.track[:, 1] - self.track[:, 0]
        self._start_pose = torch.cat([self.track[:, 0], torch.atan2(-d[:, 0], d[:, 1])[:, None]], 1).contiguous()     # [K, 3]
        self._episodes = torch.zeros(n_envs, dtype=torch.int32, device=self.device)
        self._spare = None
        self.seed = int(seed)

    # ---- state ---------------------------------------------------------------------------------------------------------
    def _sample_state(self, n):
        K = self.track.shape[0]
        tid = torch.randint(0, K, (n,), device=self.device, generator=self.gen)
        s = torch.zeros(n, HDR + self.tiles, device=self.device)
        p0, p1 = self.track[tid, 0], self.track[tid, 1]
        d = p1 - p0
        s[:, 0:2] = p0
        s[:, 2] = torch.atan2(-d[:, 0], d[:, 1])          # forward = (−sin, cos)
        s[:, 12] = tid.float()
        return s

    def _frames(self, s):
        ang = s[:, 2]
        fwd = torch.stack([-torch.sin(ang), torch.cos(ang)], 1)
        side = torch.stack([torch.cos(ang), torch.sin(ang)], 1)
        return fwd, side

    def _observe(self, s):
        obs = torch.cat([s[:, :12], torch.linalg.vector_norm(s[:, 3:5], dim=1, keepdim=True)], 1)
        if self.lookahead:
            tr = self.track[s[:, 12].long()]                                    # [N, T, 2]
            near = ((tr - s[:, None, 0:2]) ** 2).sum(-1).argmin(1)
            idx = (near[:, None] + (1 + torch.arange(self.lookahead, device=self.device)) * self.lookahead_stride) % self.tiles
            rel = torch.gather(tr, 1, idx[..., None].expand(-1, -1, 2)) - s[:, None, 0:2]
            fwd, side = self._frames(s)
            obs = torch.cat([obs, torch.stack([(rel * side[:, None]).sum(-1), (rel * fwd[:, None]).sum(-1)], -1).flatten(1)], 1)
        return obs

    # ---- one step ------------------------------------------------------------------------------------------------------
    def _dynamics(self, s, a):
        if self.use_kernels and s.is_cuda:
            return self._dynamics_kernel(s, a)
        return self._dynamics_tensor(s, a)

    # ---- the whole environment step as one kernel (CUDA) -----------------------------------------------------------------
    @property
    def graph_safe(self) -> bool:
        return self.use_kernels and self.device.type == "cuda"   # one in-place launch with a counter-hash generator

    def _fused(self) -> bool:
        return self.use_kernels and self.device.type == "cuda" and self.state is not None

    def step(self, action, reward, done, terminated, obs_f32=None, obs_bf16=None, next_obs_f32=None, next_obs_bf16=None,
             finished_return=None, do_reset=True, ep_stats=None, dbg=None):
        """Engine-style step into caller-owned buffers.  On CUDA this is ONE launch: dynamics, reward, time limit, episode
        statistics, both observations (fp32 and / or padded bf16 rows) and the reset, whose new track comes from a counter
        hash of (seed, lane, episode)."""
        if not self._fused():
            return super().step(action, reward, done, terminated, obs_f32, obs_bf16, next_obs_f32, next_obs_bf16, finished_return,
                                do_reset, ep_stats, dbg)
        from .._native import check, cuda_lib, ptr, stream_ptr
        c = ctypes
        assert action.dtype == torch.float32 and action.stride(-1) == 1 and self.state.is_contiguous()
        if self._spare is None or self._spare.shape != self.state.shape:
            self._spare = torch.empty_like(self.state)
        out, pre = self.state, self._spare                       # in place: a captured rollout keeps its addresses
        ld16 = (obs_bf16 if obs_bf16 is not None else next_obs_bf16).stride(0) if (obs_bf16 is not None or next_obs_bf16 is not None) else 0
        check(cuda_lib().nb_car_env_step(
            ptr(self.state), ptr(out), ptr(pre), ptr(action), c.c_int(action.stride(0)), ptr(self.track), c.c_int(self.tiles),
            c.c_int(self.track.shape[0]), ptr(self._start_pose), ptr(self.steps), ptr(self.ep_return), ptr(self._episodes), ptr(reward),
            ptr(done), ptr(terminated), ptr(finished_return), ptr(ep_stats), ptr(obs_f32), ptr(next_obs_f32), ptr(obs_bf16),
            ptr(next_obs_bf16), c.c_int(ld16), c.c_int(self.n_envs), c.c_int(self.obs_dim), c.c_int(self.lookahead),
            c.c_int(self.lookahead_stride), c.c_int(self.max_steps), c.c_int(1 if do_reset else 0), c.c_uint(self.seed & 0xFFFFFFFF),
            self._cparams, stream_ptr()), "car_env_step")
        self.pre_reset_state = pre

    def step_batch(self, action, auto_reset: bool = True):
        if not self._fused():
            return super().step_batch(action, auto_reset)
        a = action.to(self.device, torch.float32)
        a = a if (a.dim() == 2 and a.stride(-1) == 1) else a.reshape(self.n_envs, -1).contiguous()
        self.step(a, self.reward, self.done, self.terminated, obs_f32=self.obs, next_obs_f32=self.next_obs,
                  finished_return=self.finished_return, do_reset=auto_reset, ep_stats=self.ep_stats)
        return self.obs, self.reward, self.done, self.terminated

    def _dynamics_kernel(self, s, a):
        from .._native import check, cuda_lib, ptr, stream_ptr
        s = s.contiguous()
        a = a.contiguous()
        out, r, term = torch.empty_like(s), torch.empty(s.shape[0], device=s.device), torch.empty(s.shape[0], device=s.device)
        check(cuda_lib().nb_car_step(ptr(s), ptr(a), ctypes.c_int(a.shape[1]), ptr(self.track), ctypes.c_int(self.tiles), ptr(out),
                                     ptr(r), ptr(term), ctypes.c_int(s.shape[0]), self._cparams, stream_ptr()), "car_step")
        return out, r, term > 0.5

    def _dynamics_tensor(self, s, a):
        P = self.params
        dt = P["dt"]
        pos, ang, vel, om = s[:, 0:2], s[:, 2], s[:, 3:5], s[:, 5]
        joint = torch.cat([s[:, 6:8], torch.zeros_like(s[:, 6:8])], 1)          # [N, 4]
        wom = s[:, 8:12].clone()
        tr = self.track[s[:, 12].long()]
        ca, sa = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        rx, ry = ca * self._wx - sa * self._wy, sa * self._wx + ca * self._wy   # [N, 4]
        wpos = pos[:, None] + torch.stack([rx, ry], -1)                         # [N, 4, 2]
        d2 = _seg_dist2(wpos[:, :, None], tr[:, None], torch.roll(tr, -1, 1)[:, None])    # [N, 4, T]
        w2 = P["half_width"] ** 2
        on_road = d2.min(-1).values <= w2
        hit = (d2 <= w2).any(1)
        was = s[:, HDR:] != 0
        fresh = (hit & ~was).sum(1).float()
        steer, gas, brake = a[:, 0].clamp(-1, 1), a[:, 1].clamp(0, 1), a[:, 2].clamp(0, 1)
        gas_state = s[:, 14] + (gas - s[:, 14]).clamp(max=0.1)
        diff = -steer[:, None] * P["steer_limit"] - joint[:, :2]
        stepv = torch.sign(diff) * torch.minimum(P["steer_gain"] * diff.abs(), torch.full_like(diff, P["steer_speed"])) * dt
        joint = torch.cat([joint[:, :2] + torch.where(stepv.abs() > diff.abs(), diff, stepv), joint[:, 2:]], 1)
        drive = dt * P["engine_power"] * gas_state[:, None] / P["wheel_moment"] / (wom[:, 2:].abs() + 5.0)
        wom = torch.cat([wom[:, :2], wom[:, 2:] + drive], 1)
        val = torch.minimum(P["brake_force"] * brake[:, None], wom.abs())
        braked = wom - torch.sign(wom) * val
        wom = torch.where(brake[:, None] >= 0.9, torch.zeros_like(wom), torch.where(brake[:, None] > 0, braked, wom))
        wa = ang[:, None] + joint
        cw, sw = torch.cos(wa), torch.sin(wa)
        pvx, pvy = vel[:, 0:1] - om[:, None] * ry, vel[:, 1:2] + om[:, None] * rx
        vf, vs = -sw * pvx + cw * pvy, cw * pvx + sw * pvy
        ff, pf = (-vf + wom * P["wheel_radius"]) * P["friction_coef"], -vs * P["friction_coef"]
        lim = P["friction_limit"] * torch.where(on_road, 1.0, P["grass_friction"])
        mag = torch.sqrt(ff * ff + pf * pf)
        k = torch.where(mag > lim, lim / mag.clamp_min(1e-20), torch.ones_like(mag))
        ff, pf = ff * k, pf * k
        wom = wom - dt * ff * P["wheel_radius"] / P["wheel_moment"]
        gx, gy = pf * cw - ff * sw, pf * sw + ff * cw
        vel2 = vel + dt * torch.stack([gx.sum(1), gy.sum(1)], 1) / P["hull_mass"]
        om2 = om + dt * (rx * gy - ry * gx).sum(1) / P["hull_inertia"]
        pos2 = pos + dt * vel2
        visited = s[:, 13] + fresh
        out = (pos2.abs() > P["playfield"]).any(1)
        lap = visited >= P["lap_fraction"] * self.tiles
        hdr = torch.cat([pos2, (ang + dt * om2)[:, None], vel2, om2[:, None], joint[:, :2], wom, s[:, 12:13], visited[:, None],
                         gas_state[:, None], s[:, 15:16]], 1)
        s2 = torch.cat([hdr, (hit | was).float()], 1)
        r = torch.where(out, torch.full_like(fresh, -100.0), -0.1 + P["tile_reward"] * fresh)
        return s2, r, out | lap

    # ---- camera --------------------------------------------------------------------------------------------------------
    def render(self, res: int = 96, state=None, uint8: bool = False) -> torch.Tensor:
        """Ego-centric grey-scale image [N, res, res]: the car at (res / 2, 3 res / 4) heading up, Gymnasium's zoom
        (2.7 · 6 pixels per unit in a 1000-pixel window, scaled to ``res``).  fp32 values 0.3 / 0.7 / 1.0, or with ``uint8``
        the bytes 77 / 179 / 255 (a quarter of the memory traffic, what a replay buffer of frames stores)."""
        s = self.state if state is None else state
        ppu, cy = 2.7 * SCALE * res / 1000.0, 0.75 * res
        if self.use_kernels and s.is_cuda:
            from .._native import check, cuda_lib, ptr, stream_ptr
            s = s.contiguous()
            img = torch.empty(s.shape[0], res, res, device=s.device, dtype=torch.uint8 if uint8 else torch.float32)
            c_f = ctypes.c_float
            check(cuda_lib().nb_car_render(ptr(s), ctypes.c_int(s.shape[1]), ptr(self.track), ctypes.c_int(self.tiles), ptr(img),
                                           ctypes.c_int(s.shape[0]), ctypes.c_int(res), c_f(ppu), c_f(cy), c_f(self.params["half_width"]),
                                           c_f(CAR_HW), c_f(CAR_HL), ctypes.c_int(1 if uint8 else 0), stream_ptr()), "car_render")
            return img
        img = self._render_tensor(s, res, ppu, cy)
        return (img * 255.0 + 0.5).to(torch.uint8) if uint8 else img

    def _render_tensor(self, s, res, ppu, cy):
        dev = s.device
        jj = (torch.arange(res, device=dev) + 0.5 - 0.5 * res) / ppu
        ii = (cy - (torch.arange(res, device=dev) + 0.5)) / ppu
        ly, lx = torch.meshgrid(ii, jj, indexing="ij")
        lx, ly = lx.reshape(-1), ly.reshape(-1)
        ca, sa = torch.cos(s[:, 2])[:, None], torch.sin(s[:, 2])[:, None]
        q = torch.stack([s[:, 0:1] + ca * lx - sa * ly, s[:, 1:2] + sa * lx + ca * ly], -1)      # [N, P, 2]
        tr = self.track[s[:, 12].long()]
        road = torch.zeros(s.shape[0], res * res, dtype=torch.bool, device=dev)
        w2 = self.params["half_width"] ** 2
        for c in range(0, self.tiles, 32):          # chunks of tiles bound the [N, P, chunk] intermediate
            a, b = tr[:, None, c:c + 32], torch.roll(tr, -1, 1)[:, None, c:c + 32]
            road |= (_seg_dist2(q[:, :, None], a, b) <= w2).any(-1)
        img = torch.where(road, 0.7, 0.3)
        car = (lx.abs() <= CAR_HW) & (ly.abs() <= CAR_HL)
        return torch.where(car[None], torch.ones_like(img), img).reshape(-1, res, res)

    def visited_fraction(self) -> torch.Tensor:
        return self.state[:, 13] / self.tiles


def scripted_driver(env: CarRacingEnv, target_speed: float = 40.0, ahead: int = 5) -> torch.Tensor:
    """A pure-pursuit driver (noeira/envs/car_racing/scripted_driver.mojo has the reference's): steer toward a tile a
    few tiles ahead, gas below the target speed, brake when far above it or when the turn is sharp."""
    s = env.state
    tr = env.track[s[:, 12].long()]
    near = ((tr - s[:, None, 0:2]) ** 2).sum(-1).argmin(1)
    tgt = torch.gather(tr, 1, ((near + ahead) % env.tiles)[:, None, None].expand(-1, 1, 2))[:, 0] - s[:, 0:2]
    fwd, side = env._frames(s)
    lx, ly = (tgt * side).sum(1), (tgt * fwd).sum(1)
    bearing = torch.atan2(lx, ly.clamp_min(1e-3))                       # + = target to the right
    speed = torch.linalg.vector_norm(s[:, 3:5], dim=1)
    want = target_speed / (1.0 + 2.5 * bearing.abs())
    steer = (bearing * 2.5).clamp(-1, 1)
    gas = ((want - speed) * 0.3).clamp(0, 1)
    brake = ((speed - want - 4.0) * 0.1).clamp(0, 0.8)
    return torch.stack([steer, gas, brake], 1)


DISCRETE_TABLE = ((0.0, 0.0, 0.0), (-1.0, 0.0, 0.0), (1.0, 0.0, 0.0), (0.0, 1.0, 0.0), (0.0, 0.0, 0.8))   # noop left right gas brake


def CarRacingDiscreteEnv(n_envs: int, device="cpu", seed: int = 0, **kw):
    """Five discrete actions over the continuous environment (noeira/envs/car_racing/car_racing_discrete.mojo)."""
    return DiscreteActions(CarRacingEnv(n_envs, device, seed, **kw), DISCRETE_TABLE)


class CarRacingPixelEnv:
    """Image observations: ``stack`` grey-scale frames of ``res × res`` (newest last), five discrete actions
    (noeira/envs/car_racing/car_racing_pixel.mojo).  ``obs`` is [N, stack, res, res]; a lane that resets starts with its
    first frame repeated."""

    def __init__(self, n_envs: int, device="cpu", seed: int = 0, res: int = 64, stack: int = 4, **kw):
        self.env = CarRacingEnv(n_envs, device, seed, **kw)
        self.table = torch.tensor(DISCRETE_TABLE, device=self.env.device)
        self.n_envs, self.device, self.res, self.stack, self.n_actions = n_envs, self.env.device, res, stack, len(DISCRETE_TABLE)
        self.obs = torch.zeros(n_envs, stack, res, res, device=self.device)
        self.next_obs = torch.zeros_like(self.obs)

    def __getattr__(self, k):
        return getattr(self.env, k)

    def reset_batch(self):
        self.env.reset_batch()
        self.obs.copy_(self.env.render(self.res)[:, None].expand(-1, self.stack, -1, -1))
        return self.obs

    def step_batch(self, a, auto_reset: bool = True):
        env = self.env
        _, reward, done, terminated = env.step_batch(self.table[a.long().reshape(-1)], auto_reset=auto_reset)
        self.next_obs.copy_(torch.cat([self.obs[:, 1:], env.render(self.res, env.pre_reset_state)[:, None]], 1))
        frame = env.render(self.res)
        fresh = (done > 0.5) if auto_reset else torch.zeros_like(done, dtype=torch.bool)
        rolled = torch.cat([self.obs[:, 1:], frame[:, None]], 1)
        self.obs.copy_(torch.where(fresh[:, None, None, None], frame[:, None].expand(-1, self.stack, -1, -1), rolled))
        return self.obs, reward, done, terminated
