"""Predictive coding: inference descends the energy, local gradients agree with back-propagation in the small-error limit,
training fits a function, the stabilisers bound what they should."""
import torch

from noeira_b200.experimental.pcn import PCSequential, PCTrainer, clip_grad_norm, spectral_norm_clamp


def _data(n=128, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.rand(n, 2, generator=g) * 2 - 1
    return x, torch.stack([torch.sin(2 * x[:, 0]) * x[:, 1], x[:, 0] ** 2 - 0.5], 1)


def test_inference_descends_the_energy_and_feedforward_state_has_none():
    net = PCSequential([2, 16, 16, 2], act="tanh", seed=0)
    tr = PCTrainer(net, infer_steps=40, infer_lr=0.1)
    x, y = _data()
    assert float(net.energy(net.forward(x))) < 1e-12
    trace = []
    tr.infer(x, y, trace=trace)
    assert all(b <= a + 1e-9 for a, b in zip(trace, trace[1:])) and trace[-1] < 0.7 * trace[0]
    # without a target the feed-forward state is already the minimum: nothing moves
    xs = tr.infer(x)
    assert all((a - b).abs().max() < 1e-6 for a, b in zip(xs, net.forward(x)))


def test_local_gradients_approach_backprop_under_a_weak_output_clamp():
    for act in ("tanh", "swish", "relu"):
        x, y = _data(64, seed=1)
        seen = {}
        for lam in (1.0, 1e-3):
            net = PCSequential([2, 12, 10, 2], act=act, seed=1)
            tr = PCTrainer(net, infer_steps=300, infer_lr=0.05, output_precision=lam)
            xs = tr.infer(x, y)
            tr.opt.zero_grad()
            tr.local_grads(xs)
            ws = [blk.w.data.clone().requires_grad_(True) for blk in net.blocks]
            bs = [blk.b.data.clone().requires_grad_(True) for blk in net.blocks]
            h = x
            for blk, w, b in zip(net.blocks, ws, bs):
                h = blk.f(h) @ w.T + b
            (0.5 * (h - y).pow(2).sum(1).mean()).backward()
            cos, ratio = [], []
            for blk, w, b in zip(net.blocks, ws, bs):
                for got, want in ((blk.w.grad / lam, w.grad), (blk.b.grad / lam, b.grad)):
                    cos.append(float((got * want).sum() / (got.norm() * want.norm()).clamp_min(1e-30)))
                    ratio.append(float(got.norm() / want.norm()))
            seen[lam] = (min(cos), min(ratio), max(ratio))
        assert seen[1e-3][0] > 0.9999 and 0.97 < seen[1e-3][1] and seen[1e-3][2] < 1.01, (act, seen)
        assert seen[1.0][0] > 0.5 and seen[1.0][2] < 1.0, (act, seen)          # a descent direction, shorter


def test_training_fits_a_function_through_the_arena_optimizer():
    net = PCSequential([2, 32, 32, 2], act="tanh", seed=2)
    tr = PCTrainer(net, lr=3e-3, infer_steps=15, infer_lr=0.1, max_grad_norm=5.0, max_spectral_norm=4.0)
    x, y = _data(256, seed=2)
    first = float(tr.readout_loss(x, y))
    for _ in range(400):
        tr.train_step(x, y)
    assert float(tr.readout_loss(x, y)) < 0.2 * first
    xt, yt = _data(256, seed=9)
    assert float(tr.readout_loss(xt, yt)) < 0.3 * first


def test_stabilisers():
    g = torch.Generator().manual_seed(0)
    w = torch.randn(20, 30, generator=g)
    top = float(torch.linalg.svdvals(w)[0])
    found = spectral_norm_clamp(w, 2.0)
    assert abs(found - top) < 1e-2 * top and abs(float(torch.linalg.svdvals(w)[0]) - 2.0) < 0.03
    small = torch.eye(4) * 0.5
    spectral_norm_clamp(small, 2.0)
    assert torch.equal(small, torch.eye(4) * 0.5)
    net = PCSequential([2, 4, 2])
    ps = [p for _, p in net.named_params()]
    for p in ps:
        p.grad.fill_(1.0)
    n = clip_grad_norm(ps, 1.0)
    assert n > 1 and abs(sum(float(p.grad.pow(2).sum()) for p in ps) - 1.0) < 1e-5
