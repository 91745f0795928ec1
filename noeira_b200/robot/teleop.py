"""Leader / follower teleoperation, episode recording and policy deployment on servo arms.

``ArmBus``        joint-level view of a ``FeetechBus``: ids, calibration (centre ticks, sign, limits), ``read_joints()`` in
                  radians, ``write_joints(q)`` with limit clamping through one sync-write
``TeleopSession`` one control tick = read the leader's joints, optionally low-pass and rate-limit them, command the follower,
                  grab the newest camera frames; with a recorder attached every tick becomes a dataset row
                  (state = follower joints, action = commanded joints, one image per camera)
``EpisodeRecorder``  buffers the rows of an episode and writes an ALOHA-style HDF5 file (``data.act_dataset.save_aloha_episode``)
``run_policy``    the deployment loop of a chunked policy: a ``VLAQueryWorker`` (or any callable) turns observations into action
                  chunks off the control thread, a ``ChunkCursor`` feeds one action per tick to the follower
All of it is hardware-free by construction: the buses only need ``read_position`` / ``sync_write_positions``, the cameras
``take_latest()``, so the tests run against in-memory fakes and the serial pty loopback.
(noeira/robot/: so101 leader / follower drivers, teleop and record loops.)
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np

from .feetech import radians_to_ticks, ticks_to_radians


@dataclass
class JointCalibration:
    servo_id: int
    centre: int = 2048
    sign: int = 1
    lower: float = -3.14
    upper: float = 3.14


class ArmBus:
    def __init__(self, bus, joints: Sequence[JointCalibration]):
        self.bus, self.joints = bus, list(joints)

    def read_joints(self) -> np.ndarray:
        return np.array([j.sign * ticks_to_radians(self.bus.read_position(j.servo_id), j.centre) for j in self.joints], np.float32)

    def write_joints(self, q) -> np.ndarray:
        q = np.clip(np.asarray(q, np.float32), [j.lower for j in self.joints], [j.upper for j in self.joints])
        self.bus.sync_write_positions({j.servo_id: radians_to_ticks(j.sign * float(v), j.centre) for j, v in zip(self.joints, q)})
        return q


class EpisodeRecorder:
    def __init__(self, cameras: Sequence[str]):
        self.cameras = list(cameras)
        self.reset()

    def reset(self):
        self.qpos, self.action, self.images = [], [], {c: [] for c in self.cameras}

    def add(self, qpos, action, frames: Dict[str, np.ndarray]):
        self.qpos.append(np.asarray(qpos, np.float32))
        self.action.append(np.asarray(action, np.float32))
        for c in self.cameras:
            self.images[c].append(np.asarray(frames[c], np.uint8))

    def __len__(self):
        return len(self.qpos)

    def episode(self) -> dict:
        import torch
        img = np.stack([np.stack(self.images[c]) for c in self.cameras], 1) if self.cameras else np.zeros((len(self), 0, 1, 1, 3), np.uint8)
        return dict(qpos=torch.from_numpy(np.stack(self.qpos)), action=torch.from_numpy(np.stack(self.action)),
                    images=torch.from_numpy(img).permute(0, 1, 4, 2, 3).contiguous())           # [T, cams, 3, H, W]

    def save(self, path: str):
        from ..data.act_dataset import save_aloha_episode
        save_aloha_episode(path, self.episode(), self.cameras)


class TeleopSession:
    def __init__(self, leader: ArmBus, follower: ArmBus, cameras: Optional[Dict[str, object]] = None, rate_hz: float = 50.0,
                 smoothing: float = 0.0, max_step: float = 0.0, recorder: Optional[EpisodeRecorder] = None, clock=time.monotonic,
                 sleep=time.sleep):
        self.leader, self.follower, self.cameras = leader, follower, cameras or {}
        self.period, self.smoothing, self.max_step = 1.0 / rate_hz, smoothing, max_step
        self.recorder, self.clock, self.sleep = recorder, clock, sleep
        self._cmd = None
        self._frames: Dict[str, np.ndarray] = {}
        self.ticks = self.overruns = 0

    def _grab(self):
        for name, cam in self.cameras.items():
            f = cam.take_latest()
            if f is not None:
                self._frames[name] = f[0] if isinstance(f, tuple) else f
        return self._frames

    def tick(self) -> np.ndarray:
        target = self.leader.read_joints()
        if self._cmd is None:
            self._cmd = self.follower.read_joints()
        cmd = self.smoothing * self._cmd + (1 - self.smoothing) * target
        if self.max_step > 0:
            cmd = self._cmd + np.clip(cmd - self._cmd, -self.max_step, self.max_step)
        state = self.follower.read_joints()
        self._cmd = self.follower.write_joints(cmd)
        frames = self._grab()
        if self.recorder is not None and all(c in frames for c in self.recorder.cameras):
            self.recorder.add(state, self._cmd, frames)
        self.ticks += 1
        return self._cmd

    def run(self, n_ticks: int, stop: Optional[Callable[[], bool]] = None):
        nxt = self.clock()
        for _ in range(n_ticks):
            if stop is not None and stop():
                break
            self.tick()
            nxt += self.period
            left = nxt - self.clock()
            if left > 0:
                self.sleep(left)
            else:
                self.overruns += 1
                nxt = self.clock()


def run_policy(follower: ArmBus, cameras: Dict[str, object], worker, n_ticks: int, rate_hz: float = 30.0, requery_every: int = 10,
               observe: Optional[Callable] = None, clock=time.monotonic, sleep=time.sleep) -> List[np.ndarray]:
    """Deployment loop: every ``requery_every`` ticks the newest observation goes to ``worker.submit``; finished chunks are
    offered to a ``ChunkCursor`` stamped with the tick of their observation; the follower executes one action per tick
    (it holds its pose until the first chunk arrives).  Returns the commanded joint vectors."""
    from ..models.vla_worker import ChunkCursor
    cur, sent, out, submitted_at = ChunkCursor(), 0, [], {}
    period, nxt = 1.0 / rate_hz, clock()
    for tick in range(n_ticks):
        q = follower.read_joints()
        if tick % requery_every == 0:
            frames = {n: (c.take_latest()) for n, c in cameras.items()}
            obs = observe(q, frames) if observe is not None else (q, frames)
            seq = worker.submit(*obs) if isinstance(obs, tuple) else worker.submit(obs)
            submitted_at[seq] = tick
        res = worker.latest()
        if res is not None and res[0] > sent:
            sent = res[0]
            cur.offer(np.asarray(res[1]), submitted_at.get(res[0], tick))
        a = cur.action(tick)
        out.append(follower.write_joints(a if a is not None else q))
        nxt += period
        left = nxt - clock()
        if left > 0:
            sleep(left)
    return out
