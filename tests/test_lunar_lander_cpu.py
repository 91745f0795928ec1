"""LunarLander on the 2-D rigid-body core (host build of the source the CUDA kernel runs)."""
import torch


def _env(n=16, seed=0):
    from noeira_b200.envs.lunar_lander import LunarLanderEnv
    return LunarLanderEnv(n, device="cpu", seed=seed)


def test_reset_observation_and_free_fall():
    env = _env()
    obs = env.reset_batch().clone()
    assert obs.shape == (16, 8) and torch.isfinite(obs).all()
    assert torch.allclose(obs[:, 0], torch.zeros(16), atol=1e-6)       # starts above the middle of the view
    assert (obs[:, 1] > 1.3).all() and (obs[:, 6:] == 0).all()
    pose0 = env.lander_pose()
    zero = torch.zeros(16, 2)
    for _ in range(10):
        env.step_batch(zero)
    pose = env.lander_pose()
    # no thrust: the hull shares its initial push with the two legs it drags along (momentum is conserved),
    # vertical velocity follows gravity
    share = 4.816667 / (4.816667 + 2 * 0.071111)
    assert torch.allclose(pose[:, 3], pose0[:, 3] * share, atol=0.02)
    assert torch.allclose(pose[:, 4] - pose0[:, 4] * share, torch.full((16,), -10.0 * 10 / 50.0), atol=0.05)
    assert (env.reward.abs() < 10).all() and (env.done == 0).all()


def test_main_engine_lifts_and_costs_fuel():
    a, b = _env(8, seed=3), _env(8, seed=3)
    a.reset_batch(); b.reset_batch()
    up = torch.tensor([[1.0, 0.0]]).repeat(8, 1)
    for _ in range(20):
        a.step_batch(up)
        b.step_batch(torch.zeros(8, 2))
    assert (a.lander_pose()[:, 4] > b.lander_pose()[:, 4] + 1.0).all()      # main engine decelerates the fall
    side = torch.tensor([[0.0, 1.0]]).repeat(8, 1)
    c = _env(8, seed=3)
    c.reset_batch()
    for _ in range(20):
        c.step_batch(side)
    assert (c.lander_pose()[:, 5].abs() > b.lander_pose()[:, 5].abs() + 0.05).all()   # side engine spins the hull


def test_uncontrolled_descent_crashes_with_penalty_and_resets():
    env = _env(32, seed=1)
    env.reset_batch()
    finished = torch.zeros(32, dtype=torch.bool)
    rets = torch.full((32,), float("nan"))
    last = torch.full((32,), float("nan"))
    for _ in range(400):
        env.step_batch(torch.zeros(32, 2))
        d = env.done > 0
        rets = torch.where(d & ~finished, env.finished_return, rets)
        last = torch.where(d & ~finished, env.reward, last)
        # a finished lane is reset in the same step: its observation is a fresh start
        assert (env.obs[d, 1] > 1.3).all()
        finished |= d
    assert finished.all()
    assert (last == -100).all()          # free fall ends in a crash or out of view: −100 on the last step
    assert (rets < 0).all()              # which the shaping gathered on the way down never outweighs
    assert float(env.ep_stats[1]) >= 32


def test_scripted_controller_lands():
    """The classic heuristic (PID on angle and hover targets) lands on the helipad with a positive return."""
    env = _env(64, seed=5)
    obs = env.reset_batch().clone()
    finished = torch.zeros(64, dtype=torch.bool)
    rets = torch.full((64,), float("nan"))
    for _ in range(1000):
        s = obs
        angle_targ = (s[:, 0] * 0.5 + s[:, 2] * 1.0).clamp(-0.4, 0.4)
        hover_targ = 0.55 * s[:, 0].abs()
        angle_todo = (angle_targ - s[:, 4]) * 0.5 - s[:, 5] * 1.0
        hover_todo = (hover_targ - s[:, 1]) * 0.5 - s[:, 3] * 0.5
        legs = (s[:, 6] > 0) | (s[:, 7] > 0)
        angle_todo = torch.where(legs, torch.zeros_like(angle_todo), angle_todo)
        hover_todo = torch.where(legs, -s[:, 3] * 0.5, hover_todo)
        act = torch.stack([hover_todo * 20 - 1, -angle_todo * 20], dim=1).clamp(-1, 1)
        env.step_batch(act)
        d = env.done > 0
        rets = torch.where(d & ~finished, env.finished_return, rets)
        finished |= d
        obs = env.obs.clone()
        if finished.all():
            break
    assert finished.float().mean().item() > 0.9
    landed = rets[finished] > 100
    assert landed.float().mean().item() > 0.6, rets
