"""C51, A2C and discrete PPO: loss gradients against autograd, projection invariants, learning on CartPole."""
import torch


class _DiscreteCartPole:
    """Two pushes (−1 / +1) through the continuous-force CartPole, with the batched-env surface the drivers use."""

    def __init__(self, n, seed=0):
        from noeira_b200.envs import CartPoleEnv
        self.env = CartPoleEnv(n, seed=seed)
        self.n_envs, self.obs_dim, self.act_dim = n, self.env.obs_dim, 1

    def __getattr__(self, k):
        return getattr(self.env, k)

    def reset_batch(self):
        return self.env.reset_batch()

    def step_batch(self, a):
        return self.env.step_batch((a.float() * 2 - 1).reshape(-1, 1))

    def selective_reset_batch(self):
        pass


def test_c51_projection_and_gradient():
    from noeira_b200.agents.discrete import C51Config, C51Trainer, project_distribution
    sup = torch.linspace(-2, 2, 5)
    p = torch.tensor([[0.1, 0.2, 0.4, 0.2, 0.1]])
    out = project_distribution(p, torch.tensor([0.5]), torch.tensor([0.0]), sup, 1.0)
    assert abs(float(out.sum()) - 1.0) < 1e-6 and abs(float((out * sup).sum()) - min(2.0, float((p * (sup + 0.5).clamp(-2, 2)).sum()))) < 1e-5
    done = project_distribution(p, torch.tensor([1.0]), torch.tensor([1.0]), sup, 0.99)
    assert torch.allclose(done, torch.tensor([[0.0, 0.0, 0.0, 1.0, 0.0]]))              # terminal: all mass at r
    tr = C51Trainer(C51Config(hidden=16, n_atoms=11, seed=1))
    g = torch.Generator().manual_seed(0)
    s, sp = torch.randn(8, 4, generator=g), torch.randn(8, 4, generator=g)
    a, r, d = torch.randint(0, 2, (8,), generator=g), torch.randn(8, generator=g), torch.zeros(8)
    w = tr.q.mods[2].weight
    before = w.data.clone()
    with torch.no_grad():
        sel = tr.q_values(sp).argmax(1)
        target = project_distribution(torch.softmax(tr._dist(tr.q_target, sp), -1)[torch.arange(8), sel], r, d, tr.support, 0.99)
    wt = w.data.clone().requires_grad_(True)
    h = tr.q.mods[1].forward(tr.q.mods[0].forward(s)).float()
    logits = (h @ wt + tr.q.mods[2].bias.data).reshape(8, 2, 11)[torch.arange(8), a]
    ref = -(target * torch.log_softmax(logits, -1)).sum(-1).mean()
    ref.backward()
    tr.opt.max_grad_norm = tr.cfg.max_grad_norm = 0.0
    tr.opt.hyper[0] = 0.0                                       # lr 0: the step leaves the weights, the gradient was computed
    grads = {}
    orig = tr.opt.step
    tr.opt.step = lambda zero_grad=False: grads.update(g=w.grad.clone()) or orig(zero_grad=zero_grad)
    out = tr.update(s, a, r, sp, d)
    assert abs(float(out["loss"]) - float(ref)) < 1e-5 and torch.allclose(grads["g"], wt.grad, atol=1e-5)
    assert torch.equal(w.data, before)


def test_categorical_objective_gradients_match_autograd():
    from noeira_b200.agents.discrete import ppo_discrete_objective
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(32, 5, generator=g, requires_grad=True)
    act = torch.randint(0, 5, (32,), generator=g)
    old = torch.log_softmax(torch.randn(32, 5, generator=g), -1).gather(1, act[:, None])[:, 0]
    adv = torch.randn(32, generator=g)
    loss, dl, kl, cf = ppo_discrete_objective(logits.detach(), act, old, adv, 0.2, 0.01)
    lp_all = torch.log_softmax(logits, -1)
    lp = lp_all.gather(1, act[:, None])[:, 0]
    ratio = (lp - old).clamp(-20, 20).exp()
    ent = -(lp_all.exp() * lp_all).sum(-1)
    ref = -torch.minimum(ratio * adv, ratio.clamp(0.8, 1.2) * adv).mean() - 0.01 * ent.mean()
    ref.backward()
    assert abs(float(loss) - float(ref)) < 1e-6 and torch.allclose(dl, logits.grad, atol=1e-6)


def test_a2c_and_ppo_discrete_learn_cartpole_through_the_generic_driver():
    from noeira_b200.agents.discrete import A2CConfig, A2CTrainer, PPODiscreteConfig, PPODiscreteTrainer
    from noeira_b200.training.rl import run_onpolicy_train_batched
    for mk, steps, floor in ((lambda: A2CTrainer(A2CConfig(hidden=32, lr=2e-3, n_steps=8, seed=0), n_envs=16), 40_000, 40.0),
                             (lambda: PPODiscreteTrainer(PPODiscreteConfig(hidden=32, lr=2e-3, rollout_len=32, seed=0), n_envs=16), 30_000, 60.0)):
        env = _DiscreteCartPole(16, seed=0)
        tr = mk()
        log = run_onpolicy_train_batched(tr, env, steps, print_every=steps // 4, episode_sync_every=8, window_size=50,
                                         initial_fill=20.0)
        assert log.mean_returns[-1] > floor and log.mean_returns[-1] > log.mean_returns[0], (type(tr).__name__, log.mean_returns)


def test_acrobot_energy_and_discrete_wrapper():
    """Unforced Acrobot conserves its energy over an RK4 step sequence; a pumping controller swings the tip above the bar;
    the discrete-action wrapper maps indices to torques."""
    import math
    from noeira_b200.envs import AcrobotEnv, DiscreteActions
    env = AcrobotEnv(4, seed=0)
    env.reset_batch()
    env.state = torch.tensor([[1.0, 0.5, 0.0, 0.0]] * 4)

    def energy(s):
        t1, t2, d1, d2 = s.unbind(1)
        e = env
        dd1 = e.m1 * e.lc1 ** 2 + e.m2 * (e.l1 ** 2 + e.lc2 ** 2 + 2 * e.l1 * e.lc2 * torch.cos(t2)) + e.i1 + e.i2
        dd2 = e.m2 * (e.lc2 ** 2 + e.l1 * e.lc2 * torch.cos(t2)) + e.i2
        d22 = e.m2 * e.lc2 ** 2 + e.i2
        T = 0.5 * dd1 * d1 ** 2 + dd2 * d1 * d2 + 0.5 * d22 * d2 ** 2
        U = -e.m1 * e.g * e.lc1 * torch.cos(t1) - e.m2 * e.g * (e.l1 * torch.cos(t1) + e.lc2 * torch.cos(t1 + t2))
        return T + U

    e0 = energy(env.state)
    for _ in range(20):
        env.step_batch(torch.zeros(4, 1), auto_reset=False)
    assert torch.allclose(energy(env.state), e0, atol=0.1)            # one RK4 step of 0.2 s: 0.6 % drift in 4 s
    d = DiscreteActions(AcrobotEnv(8, seed=1), [[-1.0], [0.0], [1.0]])
    assert d.n_actions == 3
    obs = d.reset_batch()
    solved = torch.zeros(8, dtype=torch.bool)
    for _ in range(400):
        a = (obs[:, 4] * 0 + torch.sign(obs[:, 5])).long() + 1          # pump: torque along the second joint's velocity
        obs, r, done, term = d.step_batch(a)
        solved |= term > 0
    assert solved.float().mean() > 0.7 and obs.shape == (8, 6)
