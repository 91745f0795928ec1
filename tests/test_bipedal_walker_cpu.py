"""BipedalWalker on the 2-D core (host build): geometry at reset, lidar, limp collapse, motors, joint limits, reward
accounting, determinism."""
import math

import torch


def _env(n=8, seed=0):
    from noeira_b200.envs import BipedalWalkerEnv
    return BipedalWalkerEnv(n, device="cpu", seed=seed)


def test_reset_geometry_and_lidar():
    env = _env()
    obs = env.reset_batch().clone()
    assert obs.shape == (8, 24) and torch.isfinite(obs).all()
    assert torch.allclose(obs[:, 0], torch.zeros(8)) and torch.allclose(obs[:, 4], torch.full((8,), -0.05), atol=1e-6)
    assert torch.allclose(obs[:, 9], torch.full((8,), 0.05), atol=1e-6) and torch.allclose(obs[:, [6, 11]], torch.ones(8, 2), atol=1e-6)
    # lidar ray 0 points straight down over the flat start pad: (hull origin height − pad height) / range
    range_, pad_h = 160 / 30, 400 / 30 / 4
    y0 = pad_h + 2 * 34 / 30 + 8 / 30 + 0.02
    assert torch.allclose(obs[:, 14], torch.full((8,), (y0 - pad_h) / range_), atol=2e-3)
    assert (obs[:, 14:] > 0).all() and (obs[:, 14:] <= 1).all() and (obs[:, 15:23] >= obs[:, 14:22] - 1e-4).all()
    assert len({round(float(v), 6) for v in env.hull_pose()[:, 3]}) > 1            # the initial push differs per env


def test_limp_walker_collapses_and_pays_the_fall_penalty():
    env = _env(8, seed=1)
    env.reset_batch()
    fell = torch.zeros(8, dtype=torch.bool)
    for _ in range(400):
        _, r, d, term = env.step_batch(torch.zeros(8, 4), auto_reset=False)
        newly = (term > 0) & ~fell
        assert (r[newly] == -100.0).all()
        fell |= term > 0
        if fell.all():
            break
    assert fell.all()
    assert float(env.hull_pose()[:, 1].min()) > 2.5                                 # nothing tunnelled through the ground


def test_motors_move_the_joints_inside_their_limits_and_rewards_add_up():
    env = _env(4, seed=2)
    o0 = env.reset_batch().clone()
    a = torch.tensor([[1.0, -1.0, 1.0, -1.0]] * 4) * 0.9
    total = torch.zeros(4)
    x0 = env.hull_pose()[:, 0].clone()
    steps = 0
    for _ in range(30):
        o, r, d, term = env.step_batch(a, auto_reset=False)
        if bool(d.any()):
            break
        total += r
        steps += 1
    o = env.next_obs
    assert steps >= 10
    # hips swung forward (positive motor speed) and knees bent back, all within the joint ranges (small solver slack)
    assert (o[:, 4] > o0[:, 4] + 0.2).all() and (o[:, 6] - 1.0 < o0[:, 6] - 1.0 - 0.2).all()
    assert (o[:, [4, 9]] <= 1.1 + 0.05).all() and (o[:, [4, 9]] >= -0.8 - 0.05).all()
    assert (o[:, [6, 11]] - 1.0 <= -0.1 + 0.05).all() and (o[:, [6, 11]] - 1.0 >= -1.6 - 0.05).all()
    # reward = Δ(130 x / 30 − 5 |angle|) − torque cost: the first step only initialises the shaping
    x1, ang1 = env.hull_pose()[:, 0], env.hull_pose()[:, 2]
    shaping_first = None
    cost = 0.00035 * 80 * 0.9 * 4
    env2 = _env(4, seed=2)
    env2.reset_batch()
    env2.step_batch(a, auto_reset=False)
    xs, an = env2.hull_pose()[:, 0], env2.hull_pose()[:, 2]
    want = 130 * (x1 - xs) / 30 - 5 * (ang1.abs() - an.abs()) - cost * steps
    assert torch.allclose(total, want, atol=2e-3), (total, want)


def test_deterministic_and_auto_reset():
    a, b = _env(16, seed=5), _env(16, seed=5)
    a.reset_batch(), b.reset_batch()
    g = torch.Generator().manual_seed(0)
    episodes = 0
    for _ in range(250):
        act = torch.rand(16, 4, generator=g) * 2 - 1
        oa, ra, da, _ = a.step_batch(act)
        ob, rb, db, _ = b.step_batch(act)
        assert torch.equal(oa, ob) and torch.equal(ra, rb)
        episodes += int(da.sum())
        # after an automatic reset the observation is a fresh start state
        if bool(da.any()):
            i = int(da.argmax())
            assert abs(float(oa[i, 0])) < 1e-6 and abs(float(oa[i, 4]) + 0.05) < 1e-6
    assert episodes > 0 and torch.isfinite(a.obs).all()
    assert float(a.hull_pose()[:, 1].max()) < 12 and float(a.hull_pose()[:, 3:].abs().max()) < 60
