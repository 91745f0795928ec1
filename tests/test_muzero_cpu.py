"""MuZero-style agent: gradient of the unrolled loss against autograd, and learning on a small discrete task."""
import torch


class _Corridor:
    """N parallel 1-D corridors of length 6: action 1 moves right (reward 1 at the end, episode over), action 0 moves
    left.  Observation = one-hot position.  Optimal return 1 in five steps; episodes are cut at 12 steps."""
    n_actions, obs_dim, L = 2, 6, 6

    def __init__(self, n):
        self.n_envs = n
        self.pos = torch.zeros(n, dtype=torch.long)
        self.steps = torch.zeros(n, dtype=torch.long)
        z = torch.zeros
        self.obs, self.next_obs = z(n, 6), z(n, 6)
        self.reward, self.done, self.terminated = z(n), z(n), z(n)
        self.finished_return, self.ep_return = torch.full((n,), float("nan")), z(n)
        self.ep_stats = z(4)

    def _o(self):
        return torch.nn.functional.one_hot(self.pos, 6).float()

    def reset_batch(self):
        self.pos.zero_(); self.steps.zero_(); self.ep_return.zero_()
        self.obs.copy_(self._o())
        return self.obs

    def step_batch(self, a):
        self.pos = (self.pos + torch.where(a.long() > 0, 1, -1)).clamp(0, 5)
        self.steps += 1
        term = self.pos == 5
        trunc = (self.steps >= 12) & ~term
        self.reward.copy_(term.float())
        self.ep_return += self.reward
        d = term | trunc
        self.done.copy_(d.float()); self.terminated.copy_(term.float())
        self.next_obs.copy_(self._o())
        self.finished_return.copy_(torch.where(d, self.ep_return, torch.full_like(self.ep_return, float("nan"))))
        self.pos = torch.where(d, torch.zeros_like(self.pos), self.pos)
        self.steps = torch.where(d, torch.zeros_like(self.steps), self.steps)
        self.ep_return = torch.where(d, torch.zeros_like(self.ep_return), self.ep_return)
        self.obs.copy_(self._o())
        return self.obs, self.reward, self.done, self.terminated

    def selective_reset_batch(self):
        pass


def test_scale01_vjp_matches_autograd():
    from noeira_b200.agents.muzero import _scale01, _scale01_vjp
    torch.manual_seed(0)
    x = torch.randn(7, 9, requires_grad=True)
    dy = torch.randn(7, 9)
    _scale01(x).backward(dy)
    assert torch.allclose(_scale01_vjp(x.detach(), dy), x.grad, atol=1e-5)


def test_muzero_learns_the_corridor():
    from noeira_b200.agents.muzero import MuZeroAgent, MuZeroConfig
    env = _Corridor(16)
    cfg = MuZeroConfig(obs_dim=6, n_actions=2, latent=16, hidden=32, n_simulations=12, unroll=3, td_steps=5, batch=64, lr=3e-3,
                       discount=0.95, window=256, seed=0)
    agent = MuZeroAgent(cfg, n_envs=16)
    obs = env.reset_batch().clone()
    first, losses = None, []
    for step in range(700):
        a = agent.select_action_batched(obs)
        env.step_batch(a)
        agent.record_batch(obs, a, env.reward, env.next_obs, env.done, env.terminated)
        obs = env.obs.clone()
        m = agent.train_step()
        if m:
            losses.append(m["policy_loss"] + m["value_loss"] + m["reward_loss"])
    assert losses[-1] < losses[0]
    # greedy evaluation: the search with the learned model walks straight to the goal
    env2 = _Corridor(16)
    obs = env2.reset_batch().clone()
    agent.mcts.cfg.root_noise_frac = 0.0
    total = torch.zeros(16)
    reached = torch.zeros(16, dtype=torch.bool)
    for _ in range(6):
        a = agent.select_action_batched(obs, greedy=True)
        env2.step_batch(a)
        reached |= env2.terminated > 0
        obs = env2.obs.clone()
    assert reached.float().mean().item() >= 0.8


def test_gumbel_search_and_consistency_loss_options():
    """EfficientZero-style options: Gumbel root search for acting / targets and the latent consistency loss; the
    consistency term falls as the dynamics learn to predict the encoder's next latent."""
    from noeira_b200.agents.muzero import MuZeroAgent, MuZeroConfig
    from test_discrete_agents_cpu import _DiscreteCartPole
    env = _DiscreteCartPole(8, seed=0)
    ag = MuZeroAgent(MuZeroConfig(obs_dim=4, n_actions=2, latent=16, hidden=32, n_simulations=8, unroll=3, td_steps=5, batch=64,
                                  gumbel=True, consistency_coef=2.0, window=256, seed=0), n_envs=8)
    obs = env.reset_batch().clone()
    cons = []
    for t in range(160):
        a = ag.select_action_batched(obs)
        assert abs(float(ag._pending[0].sum(1)[0]) - 1) < 1e-5                 # the improved policy is the stored target
        nxt, r, done, term = env.step_batch(a)
        ag.record_batch(obs, a, r, env.next_obs, done, term)
        obs = nxt.clone()
        out = ag.train_step()
        if out is not None:
            cons.append(out["consistency"])
    assert len(cons) > 20 and all(c == c for c in cons)
    assert sum(cons[-5:]) / 5 < sum(cons[:5]) / 5                              # −cos decreases: latents line up
    assert cons[-1] < -0.5
