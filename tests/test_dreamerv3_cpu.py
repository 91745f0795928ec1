"""DreamerV3: categorical KL / straight-through pieces, world-model learning on Pendulum, imagination and behaviour steps."""
import torch


def test_latent_pieces():
    from noeira_b200.agents.dreamerv3 import DreamerV3Agent, DreamerV3Config, categorical_kl
    ag = DreamerV3Agent(DreamerV3Config(groups=4, classes=6, deter=16, hidden=16), n_envs=2)
    logits = torch.randn(5, 24, requires_grad=True)
    lp = ag._logp(logits)
    assert lp.shape == (5, 4, 6) and torch.allclose(lp.exp().sum(-1), torch.ones(5, 4), atol=1e-6)
    assert float(lp.detach().exp().min()) >= 0.01 / 6 - 1e-7                       # the uniform mix bounds every probability
    z = ag._sample(lp)
    assert z.shape == (5, 24) and torch.allclose(z.detach().reshape(5, 4, 6).sum(-1), torch.ones(5, 4))
    z.pow(2).sum().backward()                                             # straight-through: gradient reaches the logits
    assert logits.grad.abs().sum() > 0
    a, b = ag._logp(torch.randn(3, 24)), ag._logp(torch.randn(3, 24))
    ref = torch.distributions.kl_divergence(torch.distributions.Categorical(probs=a.exp()), torch.distributions.Categorical(probs=b.exp())).sum(-1)
    assert torch.allclose(categorical_kl(a, b), ref, atol=1e-5) and float(categorical_kl(a, a).abs().max()) < 1e-6


def test_world_model_learns_and_behaviour_runs():
    from noeira_b200.agents.dreamerv3 import DreamerV3Agent, DreamerV3Config, run_dreamerv3
    from noeira_b200.envs import PendulumEnv
    cfg = DreamerV3Config(obs_dim=3, act_dim=1, deter=48, groups=6, classes=6, hidden=48, seq_len=12, batch=12, imag_horizon=5,
                          window=512, seed=0)
    env = PendulumEnv(8, seed=0)
    ag = DreamerV3Agent(cfg, n_envs=8)
    run_dreamerv3(env, ag, total_env_steps=8 * 210, seed_steps=8 * 210)   # seed data: one truncation per env inside
    assert ag.t >= 210 and int(ag.first_buf.sum()) >= 16                   # reset rows are marked, arrival rows were added
    first = ag.train_step()
    for _ in range(60):
        last = ag.train_step()
    assert all(v == v for v in last.values()), last
    assert last["recon"] < 0.5 * first["recon"], (first, last)
    assert last["kl"] > 0 and last["reward_loss"] < first["reward_loss"]
    assert ag.wm_opt.arena.grd.abs().max().item() == 0.0 and ag.critic_opt.arena.grd.abs().max().item() == 0.0
    # imagination: shapes, and the λ-return of the imagined rollouts is finite and of the task's scale
    h, z = torch.zeros(10, cfg.deter), ag._sample(ag._logp(torch.zeros(10, cfg.groups * cfg.classes))).detach()
    with torch.no_grad():
        feats, acts, ents = ag.imagine(h, z, ag._fwd)
    assert feats.shape == (6, 10, cfg.deter + 36) and acts.shape == (5, 10, 1) and float(acts.abs().max()) <= 1.0
    assert -20.0 * cfg.imag_horizon < last["imag_return"] < 1.0
    more = run_dreamerv3(env, ag, total_env_steps=8 * 6, seed_steps=0, train_every=3)      # acting through the filter
    assert isinstance(more, list) and ag._h.abs().sum() > 0
