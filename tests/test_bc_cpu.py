"""Demonstration collection, behaviour cloning, demo-seeded SAC with interventions."""
import numpy as np
import torch


def _controller(obs):
    """Energy-free PD stabiliser that is good enough near the top and a swing-up push elsewhere (a scripted expert)."""
    c, s, w = obs[:, 0], obs[:, 1], obs[:, 2]
    th = torch.atan2(s, c)
    near = (th.abs() < 0.6).float()
    u = near * (-8.0 * th - 1.5 * w) + (1 - near) * torch.sign(w + 1e-3) * 1.0
    return (u / 2.0).clamp(-1, 1)[:, None]


def test_collect_clone_and_reload(tmp_path):
    from noeira_b200.agents.bc import BCConfig, BCTrainer, collect_demos, load_demos
    from noeira_b200.envs import PendulumEnv
    env = PendulumEnv(8, seed=0)
    path = str(tmp_path / "demos.traj")
    demos = collect_demos(env, _controller, n_episodes=8, path=path)
    assert demos["obs"].shape == (8 * 200, 3) and demos["action"].shape == (1600, 1)
    again = load_demos(path)
    assert np.allclose(again["obs"], demos["obs"]) and np.allclose(again["action"], demos["action"])
    for loss in ("mse", "nll"):
        tr = BCTrainer(BCConfig(obs_dim=3, act_dim=1, hidden=64, loss=loss, batch=128, lr=2e-3), demos["obs"], demos["action"])
        first = tr.train_epoch()
        for _ in range(25):
            last = tr.train_epoch()
        assert last < 0.5 * first, (loss, first, last)
        pred = tr.act(torch.as_tensor(demos["obs"][:256]))
        err = (pred - torch.as_tensor(demos["action"][:256])).abs().mean()
        assert float(err) < 0.25, (loss, float(err))


def test_hil_serl_batches_mix_demos_and_interventions_feed_the_demo_set():
    from noeira_b200.agents.bc import HilSerlTrainer, collect_demos
    from noeira_b200.agents.sac import SACConfig
    from noeira_b200.envs import PendulumEnv
    env = PendulumEnv(4, seed=1)
    demos = collect_demos(env, _controller, n_episodes=4)
    tr = HilSerlTrainer(SACConfig(obs_dim=3, act_dim=1, hidden=32, batch=64, seed=0), demos, capacity=2000)
    n0 = tr.n_demo
    assert n0 == 800 and tr.replay.base == 1600
    obs = env.reset_batch().float().clone()
    for t in range(40):
        a = tr.select_action(obs).float()
        expert = _controller(obs)
        intervene = (torch.arange(4) == t % 4) & (t % 5 == 0)               # the operator takes over now and then
        a = torch.where(intervene[:, None], expert, a)
        nxt, r, done, term = env.step_batch(a)
        tr.store(obs, a, r.float(), env.next_obs.float(), term.float(), intervened=intervene)
        obs = nxt.float().clone()
        m = tr.update()
    assert tr.interventions == 8 and tr.n_demo == n0 + 8
    assert tr.replay.size - tr.replay.base == 160
    assert all(torch.isfinite(torch.as_tensor(float(v))) for v in m.values())
    # the executed operator actions are in the demo part of the store
    assert torch.allclose(tr.replay.a[n0:n0 + 1], _controller(tr.replay.s[n0:n0 + 1]), atol=1e-5)
