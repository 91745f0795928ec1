import math

import torch


def _point_mass_rollout(target):
    """Double integrator in the plane: actions are accelerations, reward = −distance to the target − small effort."""
    def rollout(acts):
        K, H, _ = acts.shape
        p, v = torch.zeros(K, 2), torch.zeros(K, 2)
        ret = torch.zeros(K)
        for t in range(H):
            v = v + 0.1 * acts[:, t]
            p = p + 0.1 * v
            ret += -(p - target).norm(dim=1) - 0.01 * acts[:, t].pow(2).sum(1)
        return ret
    return rollout


def test_planners_improve_over_zero_action():
    from noeira_b200.planners import CEM, MPPI, RandomShooting
    target = torch.tensor([1.0, -0.5])
    ro = _point_mass_rollout(target)
    base = float(ro(torch.zeros(1, 20, 2)))
    for P, kw, it in ((MPPI, dict(samples=256, sigma=0.6, lam=0.5), 6), (CEM, dict(samples=256, elites=24), 5),
                      (RandomShooting, dict(samples=512), 1)):
        pl = P(ro, 20, 2, seed=0, **kw)
        a0 = pl.plan(it)
        assert a0.shape == (2,) and float(ro(pl.mean[None])) > base + 2.0, P.__name__
        assert a0[0] > 0 and a0[1] < 0, (P.__name__, a0)        # first action points at the target
        pl.shift()
        assert pl.mean.shape == (20, 2)


def test_classic_envs_dynamics_and_reset():
    from noeira_b200.envs import CartPoleEnv, MountainCarContinuousEnv, PendulumEnv
    pen = PendulumEnv(8, seed=0)
    o = pen.reset_batch()
    assert o.shape == (8, 3) and torch.allclose(o[:, 0] ** 2 + o[:, 1] ** 2, torch.ones(8), atol=1e-6)
    th0, thd0 = pen.state[:, 0].clone(), pen.state[:, 1].clone()
    pen.step_batch(torch.zeros(8, 1))
    thd1 = (thd0 + 15.0 * torch.sin(th0) * 0.05).clamp(-8, 8)
    assert torch.allclose(pen.state[:, 1], thd1, atol=1e-6) and (pen.reward <= 0).all()
    for _ in range(199):
        pen.step_batch(torch.zeros(8, 1))
    assert pen.done.all() and not pen.terminated.any() and (pen.steps == 0).all() and pen.ep_stats[1] == 8
    cp = CartPoleEnv(64, seed=1)
    cp.reset_batch()
    n = 0
    while cp.ep_stats[1] == 0 and n < 400:
        cp.step_batch(torch.ones(64, 1))                 # constant push topples the pole quickly
        n += 1
    assert 5 < n < 120 and cp.terminated.any()
    mc = MountainCarContinuousEnv(4, seed=2)
    mc.reset_batch()
    for t in range(400):                                   # energy pumping: push along the velocity
        v = mc.state[:, 1]
        mc.step_batch(torch.where(v >= 0, 1.0, -1.0)[:, None])
    assert mc.ep_stats[1] >= 4 and mc.ep_stats[0] > 4 * 50


def test_ilqr_swings_pendulum_to_target():
    from noeira_b200.planners import ILQR
    dt = 0.05

    def f(x, u):       # damped pendulum, θ = 0 hanging down
        th, thd = x[0], x[1]
        thdd = -9.81 * torch.sin(th) - 0.1 * thd + u[0]
        return torch.stack([th + dt * thd, thd + dt * thdd])

    target = torch.tensor([1.0, 0.0], dtype=torch.float64)
    cost = lambda x, u: 0.5 * dt * (1e-2 * (u * u).sum() + 0.1 * ((x - target) ** 2).sum())
    final = lambda x: 50.0 * ((x - target) ** 2).sum()
    pl = ILQR(f, cost, final, horizon=40, act_dim=1)
    X0, J0 = pl.rollout(torch.zeros(2, dtype=torch.float64), torch.zeros(40, 1, dtype=torch.float64))
    U, X, J = pl.plan(torch.zeros(2), iterations=30)
    assert J < 0.05 * float(J0) and abs(float(X[-1, 0]) - 1.0) < 0.05 and abs(float(X[-1, 1])) < 0.2
    # linear-quadratic problem: one iteration reaches the optimum (the Riccati solution)
    A, B = torch.tensor([[1.0, 0.1], [0.0, 1.0]], dtype=torch.float64), torch.tensor([[0.0], [0.1]], dtype=torch.float64)
    lin = ILQR(lambda x, u: A @ x + B @ u, lambda x, u: (x * x).sum() + 0.1 * (u * u).sum(), lambda x: 10 * (x * x).sum(), 20, 1, reg=1e-9)
    x0 = torch.tensor([1.0, 0.0])
    _, _, J1 = lin.plan(x0, iterations=1)
    _, _, J5 = lin.plan(x0, iterations=5)
    assert abs(J1 - J5) < 1e-6 * max(1.0, J5)


def test_tensor_environments_offer_the_engine_style_step():
    """What the on-policy trainer drives: ``env.engine.step`` into caller-owned reward / done rows and padded bf16
    observation rows, with the reset applied by masks (no host read inside the step)."""
    import torch
    from noeira_b200.envs import CarRacingEnv, PendulumEnv
    for env in (PendulumEnv(16, seed=0), CarRacingEnv(16, seed=0, lookahead=2)):
        env.max_steps = 5
        env.reset_batch()
        assert env.engine is env and env.obs_pad == 64 and env.graph_safe is False
        first = env.obs_bf16
        assert first.shape == (16, 64) and first.dtype == torch.bfloat16 and float(first[:, env.obs_dim:].abs().max()) == 0
        r, d, t = torch.zeros(16), torch.zeros(16), torch.zeros(16)
        ob, nb = torch.zeros(16, 64, dtype=torch.bfloat16), torch.zeros(16, 64, dtype=torch.bfloat16)
        a = torch.zeros(16, 8)                                         # padded action rows
        for k in range(5):
            env.engine.step(a, r, d, t, obs_bf16=ob, next_obs_bf16=nb, ep_stats=env.ep_stats)
            assert torch.equal(ob[:, : env.obs_dim].float(), env.obs.to(torch.bfloat16).float())
            assert torch.equal(nb[:, : env.obs_dim].float(), env.next_obs.to(torch.bfloat16).float())
        assert float(d.min()) == 1.0 and float(t.max()) == 0.0           # the time limit ended every lane, none terminated
        assert int(env.steps.max()) == 0 and float(env.ep_stats[1]) == 16 and float(env.ep_stats[3]) == 80
        assert not torch.equal(ob, nb)                                 # the row after the reset differs from the successor's
