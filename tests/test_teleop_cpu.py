"""Teleoperation, recording and policy deployment against in-memory servo buses and cameras."""
import numpy as np


class FakeBus:
    def __init__(self, ids):
        self.pos = {i: 2048 for i in ids}
        self.writes = 0

    def read_position(self, sid):
        return self.pos[sid]

    def sync_write_positions(self, targets):
        self.pos.update(targets)
        self.writes += 1


class FakeCam:
    def __init__(self, value):
        self.value, self.n = value, 0

    def take_latest(self):
        self.n += 1
        return np.full((6, 8, 3), (self.value + self.n) % 255, np.uint8)


def _arms():
    from noeira_b200.robot.teleop import ArmBus, JointCalibration
    cal = [JointCalibration(i + 1, lower=-1.0, upper=1.0, sign=1 if i % 2 == 0 else -1) for i in range(4)]
    lb, fb = FakeBus(range(1, 5)), FakeBus(range(1, 5))
    return ArmBus(lb, cal), ArmBus(fb, cal), lb, fb


def test_follower_tracks_leader_with_limits_smoothing_and_recording(tmp_path):
    from noeira_b200.data.act_dataset import load_aloha_episode
    from noeira_b200.robot.feetech import radians_to_ticks
    from noeira_b200.robot.teleop import EpisodeRecorder, TeleopSession
    leader, follower, lb, fb = _arms()
    rec = EpisodeRecorder(["top", "wrist"])
    now = [0.0]
    sess = TeleopSession(leader, follower, {"top": FakeCam(10), "wrist": FakeCam(100)}, rate_hz=50, max_step=0.2, recorder=rec,
                         clock=lambda: now[0], sleep=lambda s: now.__setitem__(0, now[0] + s))
    lb.pos[1] = radians_to_ticks(0.5)
    lb.pos[2] = radians_to_ticks(-2.0)            # joint 2 has sign −1: +2.0 rad, beyond the limit of 1.0
    sess.run(12)
    q = follower.read_joints()
    assert abs(q[0] - 0.5) < 2e-3 and abs(q[1] - 1.0) < 2e-3 and abs(q[2]) < 2e-3      # tracked, clamped, untouched
    assert abs(now[0] - 12 / 50) < 1e-9 and sess.overruns == 0 and fb.writes == 12
    acts = np.stack(rec.action)
    assert np.all(np.abs(np.diff(acts[:, 0])) <= 0.2 + 1e-6) and abs(acts[2, 0] - 0.5) < 2e-3     # rate limited: 0.2, 0.4, 0.5
    assert len(rec) == 12
    path = str(tmp_path / "episode_0.hdf5")
    rec.save(path)
    ep = load_aloha_episode(path)
    assert ep["cameras"] == ["top", "wrist"] and ep["images"].shape == (12, 2, 3, 6, 8) and ep["qpos"].shape == (12, 4)
    assert np.allclose(ep["action"].numpy(), acts, atol=1e-6)


def test_policy_deployment_loop_executes_chunks():
    import time
    from noeira_b200.models.vla_worker import VLAQueryWorker
    from noeira_b200.robot.teleop import run_policy
    _, follower, _, fb = _arms()

    def policy(q, frames):                          # ramps joint 0 upwards from wherever it is, 8 steps per chunk
        return np.stack([np.array([q[0] + 0.02 * (k + 1), 0, 0, 0], np.float32) for k in range(8)])

    w = VLAQueryWorker(policy)
    try:
        out = run_policy(follower, {"top": FakeCam(0)}, w, n_ticks=40, rate_hz=200.0, requery_every=5)
    finally:
        w.close()
    traj = np.array([o[0] for o in out])
    assert len(out) == 40 and traj[-1] > 0.15 and np.all(np.diff(traj) > -0.05)       # it moved up, roughly monotonically
    assert w.error is None
