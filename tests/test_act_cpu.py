"""ACT on CPU (tiny config): the hand-written VJP chain agrees with finite differences of the loss."""
import torch


def _tiny():
    from noeira_b200.models.act import ACTConfig
    return ACTConfig(chunk=6, n_cam=2, height=64, width=64, dim=64, heads=2, ff=96, enc_layers=1, dec_layers=2, latent=8,
                     dropout=0.0, lr=1e-3)


def _loss(model, cfg, batch, eps):
    qpos, img, act, valid = batch
    ahat, info = model.forward(qpos, img, act, valid, eps)
    v = valid[:, 2:].float()
    l1 = ((ahat - act).abs() * v[..., None]).sum() / (v.sum() * cfg.action_dim)
    mu, lv = info[:, : cfg.latent], info[:, cfg.latent:]
    kl = (-0.5 * (1 + lv - mu * mu - lv.exp())).sum(1).mean()
    return l1 + cfg.kl_weight * kl, ahat, info


def test_act_vjp_matches_finite_differences():
    from noeira_b200.models.act import ACTModel
    cfg = _tiny()
    torch.manual_seed(0)
    model = ACTModel(cfg)
    B = 2
    qpos = torch.randn(B, 6)
    img = torch.randint(0, 255, (B, 2, 3, 64, 64), dtype=torch.uint8)
    act = torch.randn(B, cfg.chunk, 6)
    valid = torch.ones(B, cfg.chunk + 2)
    valid[1, 6:] = 0
    eps = torch.randn(B, cfg.latent)
    batch = (qpos, img, act, valid)
    names = [n for n, _ in model.named_params()]
    assert "qenc.weight" in names and "feat.0.conv1.weight" in names and "hs.1.cross.q.weight" in names
    loss, ahat, info = _loss(model, cfg, batch, eps)
    v = valid[:, 2:].float()
    dahat = torch.sign((ahat - act) * v[..., None]) / (v.sum() * cfg.action_dim)
    mu, lv = info[:, : cfg.latent], info[:, cfg.latent:]
    dinfo = torch.cat([mu, 0.5 * (lv.exp() - 1)], 1) * (cfg.kl_weight / B)
    model.vjp(dahat, dinfo)
    P = dict(model.named_params())
    checks = [("ahat.0.weight", (3, 2)), ("hs.1.cross.k.weight", (5, 7)), ("memory.0.attn.v.weight", (2, 9)),
              ("src.0.weight", (100, 3)), ("latinfo.weight", (4, 1)), ("cvae.0.ffn.f1.weight", (3, 4)),
              ("qpe.queries", (2, 5)), ("tgt0.queries", (1, 3)), ("prop.weight", (2, 2)), ("feat.0.layer4.1.conv2.weight", (10, 20)),
              ("aenc.0.weight", (1, 1))]
    for name, idx in checks:
        p = P[name]
        e = 2e-3
        p.data[idx] += e
        lp = _loss(model, cfg, batch, eps)[0].item()
        p.data[idx] -= 2 * e
        lm = _loss(model, cfg, batch, eps)[0].item()
        p.data[idx] += e
        fd = (lp - lm) / (2 * e)
        g = p.grad[idx].item()
        assert abs(g - fd) < 5e-2 * max(abs(fd), abs(g), 0.05), (name, g, fd)


def test_maxpool_vjp_matches_autograd():
    import torch
    from noeira_b200 import nn
    x = torch.randn(2, 9, 11, 4).bfloat16().float().requires_grad_(True)     # bf16 grid → ties and shared maxima occur
    y = torch.nn.functional.max_pool2d(x.permute(0, 3, 1, 2), 3, 2, 1).permute(0, 2, 3, 1)
    g = torch.randn_like(y)
    y.backward(g)
    pool = nn.MaxPool2D()
    assert torch.equal(pool.forward(x.detach()), y.detach())
    assert torch.allclose(pool.vjp(g), x.grad, atol=1e-6)
