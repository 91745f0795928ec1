"""SAC / TD3 on CPU (fp32): explicit VJPs against torch autograd, and the update runs and improves Q fit."""
import math

import torch


def test_squashed_gaussian_vjp_matches_autograd():
    from noeira_b200.agents.sac import SquashedGaussian
    torch.manual_seed(0)
    B, A = 16, 6
    packed = torch.randn(B, 2 * A) * 1.5
    packed[0, A] = 5.0   # clamped ln σ → zero gradient
    z = torch.randn(B, A)
    d = SquashedGaussian(A, 0.7)
    a, lp = d.forward(packed, z)
    da, dl = torch.randn(B, A), torch.randn(B)
    g = d.vjp(da, dl)
    p = packed.clone().requires_grad_(True)
    mu, ls = p[:, :A], p[:, A:].clamp(-5, 2)
    u = mu + ls.exp() * z
    y = torch.tanh(u)
    a2 = 0.7 * y
    lp2 = (-0.5 * z * z - ls - 0.5 * math.log(2 * math.pi) - torch.log(0.7 * (1 - y * y) + 1e-6)).sum(1)
    ((a2 * da).sum() + (lp2 * dl).sum()).backward()
    assert torch.allclose(a, a2) and torch.allclose(lp, lp2, atol=1e-5)
    assert torch.allclose(g, p.grad, atol=2e-3, rtol=2e-3), (g - p.grad).abs().max()


def test_sac_update_runs_and_matches_reference_first_critic_step():
    from noeira_b200.agents.sac import SACConfig, SACTrainer
    cfg = SACConfig()
    tr = SACTrainer(cfg, "cpu")
    g = torch.Generator().manual_seed(0)
    B = cfg.batch
    s, sp = torch.randn(B, 17, generator=g), torch.randn(B, 17, generator=g)
    a = torch.rand(B, 6, generator=g) * 2 - 1
    r = torch.randn(B, generator=g)
    d = (torch.rand(B, generator=g) < 0.01).float()
    names = [n for n, _ in tr.actor.named_params()]
    assert names == ["trunk.0.weight", "trunk.0.bias", "trunk.1.weight", "trunk.1.bias", "heads.0.weight", "heads.0.bias",
                     "heads.1.weight", "heads.1.bias"]
    w_before = tr.q1.params()[0].data.clone()
    t_before = tr.q1t.params()[0].data.clone()
    m0 = tr.update(s, a, r, sp, d)
    assert all(math.isfinite(float(v)) for v in m0.values())
    assert not torch.equal(w_before, tr.q1.params()[0].data)
    # Polyak: target moved by tau toward the online net
    exp = t_before + cfg.tau * (tr.q1.params()[0].data - t_before)
    assert torch.allclose(tr.q1t.params()[0].data, exp, atol=1e-6)
    first = float(m0["critic_loss"])
    for _ in range(60):
        m = tr.update(s, a, r, sp, d)
    assert float(m["critic_loss"]) < first
    assert abs(float(tr.alpha) - 0.2) < 0.05 and float(tr.alpha) != 0.2


def test_sac_checkpoint_roundtrip(tmp_path):
    from noeira_b200.agents.sac import SACTrainer
    a, b = SACTrainer(device="cpu"), SACTrainer(device="cpu")
    for p in a.actor.params():
        p.set_(torch.randn(p.shape))
    a.total_train_steps = 123
    path = str(tmp_path / "sac.ckpt")
    a.save(path)
    b.load(path)
    assert b.total_train_steps == 123
    for pa, pb in zip(a.actor.params(), b.actor.params()):
        assert torch.equal(pa.data, pb.data)
    head = open(path, "rb").read(64)
    assert head.startswith(b"storage-ckpt v3\nP trunk.0.weight 4352 1\n")


def test_td3_update_runs():
    from noeira_b200.agents.sac import TD3Trainer
    tr = TD3Trainer(device="cpu")
    g = torch.Generator().manual_seed(1)
    B = 64
    s, sp = torch.randn(B, 17, generator=g), torch.randn(B, 17, generator=g)
    a = torch.rand(B, 6, generator=g) * 2 - 1
    r, d = torch.randn(B, generator=g), torch.zeros(B)
    w0 = tr.actor.params()[0].data.clone()
    o1 = tr.update(s, a, r, sp, d)
    assert "actor_loss" not in o1
    o2 = tr.update(s, a, r, sp, d)
    assert "actor_loss" in o2 and not torch.equal(w0, tr.actor.params()[0].data)


def test_replay_policies():
    from noeira_b200.data.replay import StoreReplay
    rb = StoreReplay(100, 3, 2, demo_prefix=10)
    for i in range(30):
        rb.store_batch(torch.full((4, 3), float(i)), torch.zeros(4, 2), torch.full((4,), float(i)), torch.zeros(4, 3), torch.zeros(4))
    assert rb.size == 100 and 10 <= rb.pos < 100
    assert (rb.s[:10] == 0).all()           # demo prefix untouched by the ring
    idx = rb.uniform_indices(64)
    assert idx.min() >= 0 and idx.max() < rb.size
    pi, w = rb.per_indices(32)
    assert w.max() == 1.0 and (w > 0).all()
    mi = rb.mixed_indices(20)
    assert (mi[:10] < 10).all() and (mi[10:] >= 10).all()
    ei = rb.ere_indices(16, 5, 10)
    assert ei.min() >= 0 and ei.max() < rb.size


def test_sac_exact_resume_is_bit_identical(tmp_path):
    """save → load into a fresh trainer → one update equals the uninterrupted run bit for bit (moments, step
    counters, bias-correction products, temperature state and target critics all travel)."""
    from noeira_b200.agents.sac import SACConfig, SACTrainer
    cfg = SACConfig(obs_dim=5, act_dim=2, hidden=32, batch=16, seed=3)
    g = torch.Generator().manual_seed(0)
    batch = lambda: (torch.randn(16, 5, generator=g), torch.rand(16, 2, generator=g) * 2 - 1, torch.randn(16, generator=g),
                     torch.randn(16, 5, generator=g), (torch.rand(16, generator=g) < 0.1).float())
    a = SACTrainer(cfg)
    for _ in range(3):
        a.update(*batch())
    path = str(tmp_path / "sac.ckpt")
    a.save(path)
    rng = a.gen.get_state().clone()
    nxt = batch()
    a.update(*nxt)
    b = SACTrainer(SACConfig(obs_dim=5, act_dim=2, hidden=32, batch=16, seed=99))
    b.load(path)
    b.gen.set_state(rng)
    b.update(*nxt)
    assert b.total_train_steps == a.total_train_steps == 4
    for (n1, p1), (n2, p2) in zip(list(a.actor.named_params()) + list(a.q1.named_params()) + list(a.q1t.named_params()),
                                  list(b.actor.named_params()) + list(b.q1.named_params()) + list(b.q1t.named_params())):
        assert torch.equal(p1.data, p2.data), n1
    assert torch.equal(a.alpha_opt.state, b.alpha_opt.state)
    # the reference's own layout (no moments, three modules) still loads, and re-warms
    a.save(path, with_moments=False)
    c = SACTrainer(SACConfig(obs_dim=5, act_dim=2, hidden=32, batch=16, seed=5))
    c.load(path)
    assert torch.equal(next(iter(c.actor.named_params()))[1].data, next(iter(a.actor.named_params()))[1].data)
    assert float(c.actor_opt.scalars()["t"]) == 0.0
