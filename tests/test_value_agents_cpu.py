import numpy as np
import torch


def test_tabular_agents_solve_gridworld():
    from noeira_b200.agents.tabular import GridWorld, TabularAgent
    for kind in ("q_learning", "sarsa", "expected_sarsa", "double_q"):
        env = GridWorld()
        ag = TabularAgent(env.n_states, env.n_actions, kind, seed=1)
        ret = ag.train(env, 600)
        assert np.mean(ret[-50:]) > 0.6, (kind, np.mean(ret[-50:]))
        s, done, steps = env.reset(), False, 0
        while not done:
            s, r, done = env.step(ag.act(s, greedy=True))
            steps += 1
        assert r == 1.0 and steps <= 12, kind


def test_dqn_gradient_and_learning_on_cartpole():
    from noeira_b200.agents.dqn import DQNConfig, DQNTrainer
    from noeira_b200.envs import CartPoleEnv
    for dueling in (False, True):
        tr = DQNTrainer(DQNConfig(hidden=32, dueling=dueling, seed=2))
        s, sp = torch.randn(16, 4), torch.randn(16, 4)
        a, r, d = torch.randint(0, 2, (16,)), torch.randn(16), torch.zeros(16)
        # explicit backward of the Huber TD loss against autograd through the same network weights
        tr.q.zero_grad()
        q = tr.q.forward(s).float()
        with torch.no_grad():
            y = r + 0.99 * tr.q_target.forward(sp).float().gather(1, tr.q.forward(sp).float().argmax(1, keepdim=True))[:, 0]
        q = tr.q.forward(s).float()
        diff = q.gather(1, a[:, None])[:, 0] - y
        dq = torch.zeros_like(q).scatter_(1, a[:, None], (diff.clamp(-1, 1) / 16)[:, None])
        tr.q.vjp(dq)
        w = tr.q.mods[0].weight
        eps = 1e-3
        i = (1, 3)
        def loss_at(delta):
            w.data[i] += delta
            w.version += 1
            qq = tr.q.forward(s).float().gather(1, a[:, None])[:, 0] - y
            l = torch.where(qq.abs() <= 1, 0.5 * qq * qq, qq.abs() - 0.5).mean().item()
            w.data[i] -= delta
            w.version += 1
            return l
        fd = (loss_at(eps) - loss_at(-eps)) / (2 * eps)
        assert abs(fd - w.grad[i].item()) < 5e-3 * max(1.0, abs(fd)), (dueling, fd, w.grad[i].item())
    # learning: discrete pushes through the continuous-force CartPole (action 0/1 → −1/+1)
    env = CartPoleEnv(16, seed=0)
    tr = DQNTrainer(DQNConfig(hidden=64, lr=1e-3, eps_decay_steps=4000, target_every=100, seed=0))
    obs = env.reset_batch().clone()
    buf = []
    for t in range(1800):
        a = tr.select_action(obs)
        env.step_batch((a.float() * 2 - 1)[:, None])
        buf.append((obs.clone(), a.clone(), env.reward.clone(), env.next_obs.clone(), env.terminated.clone()))
        obs = env.obs.clone()
        if t >= 50:
            idx = torch.randint(0, len(buf), (8,))
            S, A, R, SP, D = (torch.cat([buf[int(k)][j] for k in idx]) for j in range(5))
            tr.update(S, A, R, SP, D)
    early = env.ep_stats[0].item() / max(env.ep_stats[1].item(), 1)
    env.ep_stats.zero_()
    for t in range(300):
        a = tr.select_action(obs, explore=False)
        env.step_batch((a.float() * 2 - 1)[:, None])
        obs = env.obs.clone()
    late = env.ep_stats[0].item() / max(env.ep_stats[1].item(), 1)
    assert late > 1.4 * early and late > 30, (early, late)


def test_ddpg_is_td3_without_smoothing():
    from noeira_b200.agents.sac import DDPGTrainer, TD3Config
    tr = DDPGTrainer(TD3Config(obs_dim=3, act_dim=1, hidden=16))
    assert tr.cfg.policy_delay == 1 and tr.cfg.policy_noise == 0.0
    s, a, r, sp, d = torch.randn(8, 3), torch.rand(8, 1) * 2 - 1, torch.randn(8), torch.randn(8, 3), torch.zeros(8)
    out = tr.update(s, a, r, sp, d)
    assert "actor_loss" in out and torch.isfinite(torch.as_tensor(float(out["critic_loss"])))


def test_sac_agent_drives_pendulum_and_logs(tmp_path):
    from noeira_b200 import core
    from noeira_b200.agents.sac import SACAgent, SACConfig
    from noeira_b200.envs import PendulumEnv
    env = PendulumEnv(4, seed=0)
    agent = SACAgent(env, SACConfig(obs_dim=3, act_dim=1, hidden=32, batch=32), capacity=5000, learning_starts=200)
    with core.RunContext(str(tmp_path), "t", "sac") as run:
        m = agent.train(600, logger=run, log_every=100)
    assert agent.replay.size == 600 and all(float(v) == float(v) for v in m.values())
    rows = open(run.path("metrics.csv")).read().splitlines()
    assert len(rows) >= 3 and "critic_loss" in rows[0]
