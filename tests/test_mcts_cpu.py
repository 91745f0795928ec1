"""Batched MCTS on exact models: the search must find the rewarding branch and value it correctly."""
import torch


def _chain_model(depth=4, A=3, good=(2, 0, 1, 2)):
    """Deterministic tree MDP: state = (level, on_path flag); following ``good`` pays 1 at the last level, anything else 0.
    latent = [level, on_path]."""
    good_t = torch.tensor(good)

    def initial(obs):
        n = obs.shape[0]
        return torch.zeros(n, 2), torch.zeros(n, A), torch.zeros(n)

    def recurrent(latent, action):
        level = latent[:, 0].long()
        on = latent[:, 1] == 0                                  # 0 = still on the good path
        ok = on & (level < depth) & (action == good_t[level.clamp(max=depth - 1)])
        new_level = (level + 1).clamp(max=depth)
        reward = (ok & (new_level == depth)).float()
        new = torch.stack([new_level.float(), (~ok).float()], dim=1)
        return new, reward, torch.zeros(latent.shape[0], A), torch.zeros(latent.shape[0])

    return initial, recurrent


def test_search_finds_the_rewarding_branch():
    from noeira_b200.planners.mcts import BatchedMCTS, MCTSConfig
    initial, recurrent = _chain_model()
    cfg = MCTSConfig(n_actions=3, n_simulations=400, discount=1.0, max_depth=8)
    mcts = BatchedMCTS(cfg, initial, recurrent, use_kernels=False)
    policy, value, action = mcts.search(torch.zeros(5, 1))
    assert (action == 2).all(), (action, policy)               # first move of the good path
    assert (policy[:, 2] > 0.6).all()
    assert (value > 0.2).all()                                  # the root value rises toward 1 as the search concentrates
    t = mcts.tree
    assert int(t.n_nodes.max()) == cfg.n_simulations + 1
    assert torch.allclose(t.visit[:, 0], torch.full((5,), float(cfg.n_simulations + 1)))
    # visit counts of the root's children add up to the simulations
    ch = t.children[:, 0].long()
    counts = torch.where(ch >= 0, t.visit[torch.arange(5)[:, None], ch.clamp(min=0)], torch.zeros(5, 3))
    assert torch.allclose(counts.sum(-1), torch.full((5,), float(cfg.n_simulations)))


def test_priors_and_legal_mask_are_respected():
    from noeira_b200.planners.mcts import BatchedMCTS, MCTSConfig

    def initial(obs):
        n = obs.shape[0]
        return torch.zeros(n, 1), torch.tensor([[0.0, 3.0, 0.0, 0.0]]).repeat(n, 1), torch.zeros(n)

    def recurrent(latent, action):
        n = latent.shape[0]
        return latent + 1, torch.zeros(n), torch.zeros(n, 4), torch.zeros(n)

    cfg = MCTSConfig(n_actions=4, n_simulations=60, max_depth=6)
    m = BatchedMCTS(cfg, initial, recurrent, use_kernels=False)
    legal = torch.tensor([[True, False, True, True]]).repeat(3, 1)
    policy, _, action = m.search(torch.zeros(3, 1), legal=legal)
    assert (policy[:, 1] == 0).all() and (action != 1).all()   # the strong prior sits on an illegal move: never visited
    policy2, _, action2 = m.search(torch.zeros(3, 1))
    assert (action2 == 1).all() and (policy2[:, 1] > 0.5).all()   # without the mask the prior wins (all values equal)


def test_temperature_sampling_follows_visit_counts():
    from noeira_b200.planners.mcts import BatchedMCTS, MCTSConfig
    initial, recurrent = _chain_model()
    m = BatchedMCTS(MCTSConfig(n_actions=3, n_simulations=300, discount=1.0, max_depth=8), initial, recurrent, use_kernels=False)
    g = torch.Generator().manual_seed(0)
    _, _, a = m.search(torch.zeros(256, 1), temperature=1.0, generator=g)
    assert (a == 2).float().mean() > 0.5 and (a != 2).any()


def test_gumbel_search_improves_the_policy_with_few_simulations():
    """A bandit behind a one-step model: arm rewards are known to the model, the prior is uniform.  With 16 simulations over
    8 arms the Gumbel search must return the best arm (greedy) and an improved policy that ranks the arms by reward."""
    from noeira_b200.planners.mcts import BatchedMCTS, MCTSConfig
    n, A = 32, 8
    g = torch.Generator().manual_seed(0)
    arm = torch.rand(n, A, generator=g)

    def initial(obs):
        return obs, torch.zeros(n, A), torch.zeros(n)

    def recurrent(latent, action):
        r = latent[torch.arange(latent.shape[0]), action.long()] * (latent[:, -1] == 0).float()    # reward on the first move only
        nxt = latent.clone()
        nxt[:, -1] = 1.0
        return nxt, r, torch.zeros(latent.shape[0], A), torch.zeros(latent.shape[0])

    obs = torch.cat([arm, torch.zeros(n, 1)], 1)
    mcts = BatchedMCTS(MCTSConfig(n_actions=A, n_simulations=16, discount=1.0, gumbel_considered=8, max_depth=17), initial, recurrent,
                       use_kernels=False)
    pol, val, act = mcts.search_gumbel(obs, greedy=True)
    assert (act == arm.argmax(1)).all()
    assert torch.allclose(pol.sum(1), torch.ones(n), atol=1e-5)
    assert (pol.argmax(1) == arm.argmax(1)).float().mean() > 0.9
    # with noise the chosen arm is still a good one on average, and different trees explore differently
    pol2, _, act2 = mcts.search_gumbel(obs, generator=g)
    assert float(arm[torch.arange(n), act2].mean()) > float(arm.mean()) + 0.2
    legal = torch.ones(n, A, dtype=torch.bool)
    legal[:, 0] = False
    pol3, _, act3 = mcts.search_gumbel(obs, legal=legal, greedy=True)
    assert (act3 != 0).all() and float(pol3[:, 0].max()) < 1e-6


def test_sampled_search_over_continuous_actions():
    """One-step continuous bandit: reward −(a − target)² per tree, policy N(0, 1).  Among the K sampled root actions the
    search must concentrate its visits on those nearest the target and return one of the best."""
    from noeira_b200.planners.mcts import MCTSConfig, SampledMCTS
    n, K = 16, 12
    g = torch.Generator().manual_seed(0)
    target = torch.rand(n, generator=g) * 2 - 1

    def initial(obs):
        return obs, torch.zeros(n, 2), torch.zeros(n)                       # latent = [target, moved flag]

    def recurrent(latent, action):
        first = latent[:, 1] == 0
        r = torch.where(first, -(action[:, 0] - latent[:, 0]) ** 2, torch.zeros(latent.shape[0]))
        nxt = latent.clone()
        nxt[:, 1] = 1.0
        return nxt, r, torch.zeros(latent.shape[0], 2), torch.zeros(latent.shape[0])

    def sample(params, k, gen):
        return torch.randn(params.shape[0], k, 1, generator=gen)

    obs = torch.stack([target, torch.zeros(n)], 1)
    mcts = SampledMCTS(MCTSConfig(n_actions=K, n_simulations=48, discount=1.0, max_depth=49), initial, recurrent, sample, act_dim=1,
                       use_kernels=False)
    actions, w, value, chosen = mcts.search(obs, generator=g)
    assert actions.shape == (n, K, 1) and chosen.shape == (n, 1) and torch.allclose(w.sum(1), torch.ones(n), atol=1e-5)
    err = (actions[..., 0] - target[:, None]).abs()
    # unvisited slots count as the worst value (as in MuZero), so not every sample is tried with 48 simulations: the chosen
    # action is among the better half of the samples, and the visits concentrate near the target
    assert ((chosen[:, 0] - target).abs() <= err.median(1).values + 1e-6).float().mean() > 0.85
    assert float((w * err).sum(1).mean()) < float(err.mean()) * 0.6
