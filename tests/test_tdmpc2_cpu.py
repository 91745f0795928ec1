"""Re-entrant autograd bridge, TD-MPC2 model learning and latent-space planning on Pendulum."""
import torch


def test_reentrant_bridge_matches_autograd_over_an_unroll():
    from noeira_b200 import nn
    nn.manual_seed(0)
    f = nn.Sequential(nn.LinearTanh(4, 4), nn.Linear(4, 4))
    x = torch.randn(3, 4, requires_grad=True)
    h = x
    for _ in range(3):
        h = nn.apply(f, h)                               # the same module three times in one graph
    h.pow(2).sum().backward()
    P = {n: p.data.clone().requires_grad_(True) for n, p in f.named_params()}
    xr = x.detach().clone().requires_grad_(True)
    h = xr
    for _ in range(3):
        h = torch.tanh(h @ P["0.weight"] + P["0.bias"]) @ P["1.weight"] + P["1.bias"]
    h.pow(2).sum().backward()
    assert torch.allclose(x.grad, xr.grad, atol=1e-6)
    for n, p in f.named_params():
        assert torch.allclose(p.grad, P[n].grad, atol=1e-5), n


def test_tdmpc2_learns_the_model_and_plans():
    from noeira_b200.agents.tdmpc2 import TDMPC2Agent, TDMPC2Config, run_tdmpc2, simnorm
    from noeira_b200.envs import PendulumEnv
    z = simnorm(torch.randn(5, 16), 8)
    assert torch.allclose(z.reshape(5, 2, 8).sum(-1), torch.ones(5, 2), atol=1e-6)
    cfg = TDMPC2Config(obs_dim=3, act_dim=1, latent=32, hidden=64, batch=64, horizon=3, plan_samples=48, plan_pi_samples=8,
                       plan_elites=8, plan_iterations=2, window=1024, seed=0)
    env = PendulumEnv(8, seed=0)
    ag = TDMPC2Agent(cfg, n_envs=8)
    rets = run_tdmpc2(env, ag, total_env_steps=800, seed_steps=800)          # seed data only
    first = [ag.train_step() for _ in range(5)][-1]
    for _ in range(150):
        last = ag.train_step()
    assert last["reward_loss"] < 0.5 * first["reward_loss"], (first, last)
    # the latents start near-uniform (a trivially consistent code) and become informative: the consistency term stays small
    assert last["consistency"] < 0.2 and all(v == v for v in last.values())
    assert ag.opt.arena.grd.abs().max().item() == 0.0                        # nothing left over from the policy pass
    assert not torch.equal(ag.q.params()[0].data, ag.q_target.params()[0].data)
    # planning: actions inside the bounds, a warm-started mean, and a plan whose model value is at least as good as the
    # prior's own action sequence (the prior's samples are among the candidates)
    obs = env.obs.float().clone()
    a = ag.select_action(obs, explore=False)
    assert a.shape == (8, 1) and float(a.abs().max()) <= 1.0 and ag._mean.shape == (8, 3, 1)
    with torch.no_grad():
        z0 = ag.encode(obs)
        zz, pa = z0, []
        for _ in range(cfg.horizon):
            pa.append(ag.policy(zz, sample=False))
            zz = ag.next_latent(zz, pa[-1])
        prior_val = ag._score(z0, torch.stack(pa, 1))
        plan_val = ag._score(z0, ag._mean)
    assert float((plan_val - prior_val).mean()) > -0.5
    more = run_tdmpc2(env, ag, total_env_steps=160, seed_steps=0)            # the acting loop with planning runs
    assert ag.t == 100 + 20 and isinstance(more, list)
