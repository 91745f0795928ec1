"""MBPO: ensemble loss gradients against autograd, model fit quality on Pendulum, rollouts and mixed batches."""
import torch
import torch.nn.functional as F


def test_ensemble_nll_gradients_match_autograd():
    from noeira_b200.agents.mbpo import DynamicsEnsemble, MBPOConfig
    from noeira_b200 import nn
    nn.manual_seed(0)
    cfg = MBPOConfig(obs_dim=3, act_dim=1, ensemble=4, elites=2, model_hidden=8, model_layers=2)
    m = DynamicsEnsemble(3, 1, cfg)
    g = torch.Generator().manual_seed(0)
    x, y = torch.randn(10, 4, 4, generator=g), torch.randn(10, 4, 4, generator=g)
    P = {n: p.data.clone().requires_grad_(True) for n, p in m.named_params()}
    h = x
    for i in range(3):
        W, b = P[f"net.{i}.weight"].reshape(4, -1, P[f"net.{i}.weight"].shape[1]), P[f"net.{i}.bias"].reshape(4, -1)
        h = torch.einsum("bki,kio->bko", h, W) + b
        if i < 2:
            h = F.silu(h)
    mean, raw = h[..., :4], h[..., 4:]
    lv = P["max_logvar"] - F.softplus(P["max_logvar"] - raw)
    lv = P["min_logvar"] + F.softplus(lv - P["min_logvar"])
    ref = ((mean - y) ** 2 * torch.exp(-lv) + lv).mean((0, 2)).sum() + 0.01 * (P["max_logvar"].sum() - P["min_logvar"].sum())
    ref.backward()
    mu, l2 = m.forward(x)
    loss, dm, dl = m.nll(mu, l2, y)
    m.vjp(dm, dl)
    assert abs(float(loss) - float(ref.detach())) < 1e-5
    for n, p in m.named_params():
        assert torch.allclose(p.grad, P[n].grad, atol=1e-5), n


def test_model_fits_pendulum_and_feeds_sac():
    from noeira_b200.agents.mbpo import MBPOConfig, MBPOTrainer, run_mbpo
    from noeira_b200.envs import PendulumEnv
    cfg = MBPOConfig(obs_dim=3, act_dim=1, hidden=32, batch=64, ensemble=5, elites=3, model_hidden=48, model_layers=2,
                     model_epochs=15, model_train_every=400, rollout_batch=64, rollout_len=2, real_ratio=0.25,
                     updates_per_step=2, action_scale=1.0, seed=0)
    tr = MBPOTrainer(cfg, capacity=4000)
    env = PendulumEnv(8, seed=0)
    rets = run_mbpo(env, tr, total_env_steps=1600, learning_starts=800)
    assert tr.real.size == 1600 and tr.imagined.size > 0
    assert tr.model.elite_idx.numel() == 3 and len(set(tr.model.elite_idx.tolist())) == 3
    # explained variance of the elites on fresh transitions
    s, a, r, sp, _ = tr.real.gather(torch.arange(1200, 1600))
    y = torch.cat([sp - s, r[:, None]], 1)
    mean, lv = tr.model.forward(torch.cat([s, a], 1))
    err = ((mean[:, tr.model.elite_idx].mean(1) - y) ** 2).mean(0)
    assert (err / y.var(0) < 0.2).all(), err / y.var(0)
    assert torch.isfinite(lv).all() and float(lv.max()) <= float(tr.model.max_logvar.data.max()) + 1e-4
    assert all(torch.isfinite(torch.as_tensor(float(v))) for v in tr.metrics.values())
    ns, nr = tr.model.predict(s[:16], a[:16], deterministic=True)
    assert ns.shape == (16, 3) and nr.shape == (16,)
    assert len(rets) >= 8 - 1
