"""Dreamer 4 pieces on the CPU oracle path: dynamics gradients, shortcut-forcing loss, RL losses, sampler, tokenizer."""
import math

import torch

from noeira_b200 import nn


def _fd(loss_fn, params, n=4, eps=3e-3, tol=6e-2):
    base = {name: p.grad.clone() for name, p in params}
    g = torch.Generator().manual_seed(0)
    for name, p in params:
        d, gr = p.data, base[name]
        for _ in range(n):
            i = tuple(int(torch.randint(0, s, (1,), generator=g)) for s in d.shape)
            old = d[i].item()
            d[i] = old + eps
            p.version += 1
            lp = loss_fn()
            d[i] = old - eps
            p.version += 1
            lm = loss_fn()
            d[i] = old
            p.version += 1
            fd = (lp - lm) / (2 * eps)
            assert abs(fd - gr[i].item()) < tol * max(abs(fd), abs(gr[i].item())) + 5e-4, (name, fd, gr[i].item())


def _setup(b=3, T=4, adim=0):
    from noeira_b200.agents.dreamer4 import Dreamer4Config, Dreamer4Dynamics
    cfg = Dreamer4Config(nsp=4, dsp=3, dim=16, heads=2, ff=32, depth=2, nreg=1, kmax=8, adim=adim)
    dyn = Dreamer4Dynamics(cfg, T)
    g = torch.Generator().manual_seed(1)
    BF, ND = b * T, cfg.nsp * cfg.dsp
    z1, z0 = torch.randn(BF, ND, generator=g), torch.randn(BF, ND, generator=g)
    step = torch.randint(0, cfg.emax, (BF,), generator=g)
    k = 2 ** step
    sidx = (torch.randint(0, 10 ** 6, (BF,), generator=g) % k) * (cfg.kmax // k)
    sigma = sidx.float() / cfg.kmax
    return cfg, dyn, z1, z0, sigma, sidx, step


def test_dynamics_backward_matches_finite_differences():
    cfg, dyn, z1, z0, sigma, sidx, step = _setup(adim=3)
    acts = torch.randn(z1.shape[0], 3)
    w = torch.randn_like(z1)
    wa = torch.randn(z1.shape[0] // 4, 4, cfg.dim)

    def loss():
        dyn.set_indices(sidx, step)
        dyn.set_actions(acts)
        out = dyn.forward(z0)
        return float((out * w).sum() + (dyn.agent_out() * wa).sum())
    dyn.zero_grad()
    loss()
    dyn.vjp(w, dagent=wa)
    _fd(loss, list(dyn.named_params()))
    names = [n for n, _ in dyn.named_params()]
    assert {"action_base", "signal_table", "step_table", "register", "agent_base"} <= set(names)


def test_shortcut_forcing_loss_and_gradient():
    from noeira_b200.agents.dreamer4 import shortcut_forcing_loss
    cfg, dyn, z1, z0, sigma, sidx, step = _setup(b=4)
    T, b_self = 4, 2
    loss, grad, zhat = shortcut_forcing_loss(dyn, z1, z0, sigma, sidx, step, T, b_self, cfg.kmax, do_boot=True)
    # restate the loss as a function of ẑ (targets detached) and compare its autograd gradient
    zh = zhat.detach().clone().requires_grad_(True)
    BF, ND = z1.shape
    S0 = (4 - b_self) * T
    s = sigma[:, None]
    ztil = (1 - s) * z0 + s * z1
    w = 0.9 * sigma + 0.1
    emp = (w[:S0] * (zh[:S0] - z1[:S0]).pow(2).mean(1)).sum() / S0
    # v̄ from the function's own definition: recover it through the gradient relation instead of recomputing the model
    _, g2, _ = shortcut_forcing_loss(dyn, z1, z0, sigma, sidx, step, T, b_self, cfg.kmax, do_boot=True)
    assert torch.allclose(grad, g2, atol=1e-7)                         # deterministic
    emp.backward()
    assert torch.allclose(zh.grad[:S0] * (4 - b_self) / 4, grad[:S0], atol=1e-6)   # empirical rows: closed form
    assert float(grad[S0:].abs().sum()) > 0 and torch.isfinite(loss)
    # without the bootstrap the self rows carry no loss
    l0, g0, _ = shortcut_forcing_loss(dyn, z1, z0, sigma, sidx, step, T, b_self, cfg.kmax, do_boot=False)
    assert float(g0[S0:].abs().sum()) == 0.0 and float(l0) < float(loss) + 1e-6
    # a few optimisation steps reduce the loss
    opt = nn.AdamW(dyn.named_params(), lr=3e-3)
    first = None
    for _ in range(25):
        l, g, _ = shortcut_forcing_loss(dyn, z1, z0, sigma, sidx, step, T, b_self, cfg.kmax)
        dyn.vjp(g)
        opt.step(zero_grad=True)
        first = first if first is not None else float(l)
    assert float(l) < first


def test_imagination_losses_match_autograd():
    from noeira_b200.agents.dreamer4 import continue_bce, lambda_returns, pmpo_policy_loss, value_td_loss, UNIMIX
    g = torch.Generator().manual_seed(2)
    B, H, NA, NB = 3, 5, 4, 11
    rew, val = torch.randn(B, H, generator=g), torch.randn(B, H, generator=g)
    con = 0.97 * (torch.rand(B, H, generator=g) > 0.2).float()
    ret = lambda_returns(rew, val, con, 0.9)
    for b in range(B):
        nxt = val[b, H - 1]
        for t in range(H - 2, -1, -1):
            nxt = rew[b, t + 1] + con[b, t + 1] * ((1 - 0.9) * val[b, t + 1] + 0.9 * nxt)
            assert abs(float(ret[b, t] - nxt)) < 1e-5
    bins = torch.linspace(-5, 5, NB)
    vl = torch.randn(B, H, NB, generator=g, requires_grad=True)
    loss, gv = value_td_loss(vl.detach(), ret, bins)
    from noeira_b200.nn.losses import symlog, two_hot
    ref = -(two_hot(symlog(ret.reshape(-1)), bins) * torch.log_softmax(vl[:, : H - 1].reshape(-1, NB), -1)).sum(-1).mean()
    ref.backward()
    assert abs(float(loss - ref)) < 1e-6 and torch.allclose(gv, vl.grad, atol=1e-6)
    pl = torch.randn(B, H, NA, generator=g, requires_grad=True)
    prior = torch.randn(B, H, NA, generator=g)
    acts = torch.randint(0, NA, (B, H), generator=g)
    adv = torch.randn(B, H - 1, generator=g)
    loss, gp = pmpo_policy_loss(pl.detach(), prior, acts, adv, alpha=0.4, beta=0.3)
    pm = (1 - UNIMIX) * torch.softmax(pl[:, : H - 1], -1) + UNIMIX / NA
    qm = (1 - UNIMIX) * torch.softmax(prior[:, : H - 1], -1) + UNIMIX / NA
    logp = torch.log(pm.gather(-1, acts[:, : H - 1, None]).squeeze(-1))
    pos = adv >= 0
    ref = (-(1 - 0.4) / pos.sum() * logp[pos].sum() + 0.4 / (~pos).sum() * logp[~pos].sum()
           + 0.3 / (B * (H - 1)) * (pm * (pm.log() - qm.log())).sum())
    ref.backward()
    assert abs(float(loss - ref)) < 1e-5 and torch.allclose(gp, pl.grad, atol=1e-6)
    cl = torch.randn(B, H, generator=g, requires_grad=True)
    tgt = (torch.rand(B, H, generator=g) > 0.1).float()
    loss, gc = continue_bce(cl.detach(), tgt)
    ref = torch.nn.functional.binary_cross_entropy_with_logits(cl, tgt)
    ref.backward()
    assert abs(float(loss - ref)) < 1e-6 and torch.allclose(gc, cl.grad, atol=1e-6)


def test_sampler_and_heads():
    from noeira_b200.agents.dreamer4 import continue_head, policy_head, reward_head, sample_one_timestep, value_head
    cfg, dyn, z1, z0, sigma, sidx, step = _setup(b=2)
    T, ND = 4, cfg.nsp * cfg.dsp
    ctx = z1.reshape(2, T, ND)[:, : T - 1].reshape(-1, ND)
    out = sample_one_timestep(dyn, ctx, torch.randn(2, ND), T, cfg.kmax, K=4)
    assert out.shape == (2, ND) and torch.isfinite(out).all()
    h = torch.randn(6, cfg.dim)
    assert policy_head(cfg.dim, 32, 5, 3).forward(h).shape == (6, 15)
    assert reward_head(cfg.dim, 32, 11, 3).forward(h).shape == (6, 33)
    assert value_head(cfg.dim, 32, 11).forward(h).shape == (6, 11) and continue_head(cfg.dim, 32).forward(h).shape == (6, 1)


def test_tokenizer_gradients_and_patchify_roundtrip():
    from noeira_b200.agents.dreamer4 import Dreamer4Tokenizer, downscale_box, mae_mask, temporal_patchify, temporal_unpatchify
    frames = torch.rand(2, 3, 3, 8, 12)
    p = temporal_patchify(frames, 4)
    assert p.shape == (6, 6, 48) and torch.equal(temporal_unpatchify(p, 4, 3, 8, 12, 3), frames)
    assert downscale_box(frames, 2).shape == (2, 3, 3, 4, 6)
    tok = Dreamer4Tokenizer(6, 48, nsp=2, dsp=3, dim=16, heads=2, ff=32, depth=1)
    mask = mae_mask(6, 6, 0.2, 0.6, torch.Generator().manual_seed(0))
    w = torch.randn(6, 6, 48)

    def loss():
        return float((tok.forward(p, mask) * w).sum())
    tok.zero_grad()
    loss()
    tok.vjp(w)
    _fd(loss, list(tok.named_params()), n=3, eps=2e-2, tol=8e-2)   # sigmoid outputs summed over 1.7 k pixels: wide steps keep fp32 rounding out of the quotient
    z = tok.encode(p)
    assert z.shape == (6, 6) and float(z.abs().max()) <= 1.0


def test_agent_facade_three_phases():
    """Video prediction + BC, action-conditioned world model + reward / continue heads, imagination RL with the dynamics
    frozen: losses fall on a synthetic latent process whose next frame depends on the action."""
    from noeira_b200.agents.dreamer4 import Dreamer4Agent, Dreamer4Config
    cfg = Dreamer4Config(nsp=4, dsp=4, dim=32, heads=2, ff=64, depth=1, nreg=1, kmax=4, adim=3, seed=0)
    T, B, ND = 4, 8, 16
    ag = Dreamer4Agent(cfg, T, n_actions=3, n_bins=21, head_hidden=32, lr=2e-3)
    g = torch.Generator().manual_seed(0)
    base = torch.randn(3, ND, generator=g)

    def batch():
        a = torch.randint(0, 3, (B, T), generator=g)
        z = torch.zeros(B, T, ND)
        z[:, 0] = torch.randn(B, ND, generator=g) * 0.3
        for t in range(1, T):
            z[:, t] = 0.5 * z[:, t - 1] + base[a[:, t - 1]] + 0.05 * torch.randn(B, ND, generator=g)
        rew = (a == 2).float().roll(1, 1)                                  # reward for having chosen action 2
        rew[:, 0] = 0
        return z, a, rew, torch.ones(B, T)

    first = ag.acwm_train_step(*batch())
    for _ in range(60):
        last = ag.acwm_train_step(*batch())
    assert all(v == v for v in last.values())
    assert last["wm_loss"] < first["wm_loss"] and last["reward_loss"] < first["reward_loss"] and last["cont_loss"] < first["cont_loss"]
    z, a, _, _ = batch()
    b0 = ag.bc_train_step(z, torch.full_like(a, 1))
    for _ in range(30):
        b1 = ag.bc_train_step(batch()[0], torch.full((B, T), 1))
    assert b1["bc_loss"] < 0.5 * b0["bc_loss"]                             # the policy head clones the constant demonstrator
    dyn_before = [p.data.clone() for _, p in ag.dyn.named_params()]
    ph_before = ag.ph.params()[0].data.clone()
    out = ag.imag_train_step(z, a, horizon=3, K=2)
    assert all(v == v for v in out.values()) and 0.0 <= out["imag_reward"]
    assert all(torch.equal(p.data, q) for (_, p), q in zip(ag.dyn.named_params(), dyn_before))      # dynamics frozen
    assert not torch.equal(ag.ph.params()[0].data, ph_before)
    assert [n.split(".")[0] for n, _ in ag.named_params()][0] == "dyn"
