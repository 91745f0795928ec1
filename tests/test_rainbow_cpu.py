"""NoisyLinear / BlockLinear gradients against autograd, n-step folding against a direct sum, Rainbow on CartPole."""
import torch

from test_discrete_agents_cpu import _DiscreteCartPole


def test_noisy_linear_matches_the_materialised_weight_and_autograd():
    from noeira_b200 import nn
    nn.manual_seed(0)
    lay = nn.NoisyLinear(6, 5, sigma0=0.5, out_fp32=True)
    names = [n for n, _ in lay.named_params("q.")]
    assert names == ["q.mu_w", "q.sigma_w", "q.mu_b", "q.sigma_b"]
    g = torch.Generator().manual_seed(1)
    lay.reset_noise(g)
    x = torch.randn(7, 6, generator=g)
    dy = torch.randn(7, 5, generator=g)
    P = {n: p.data.clone().requires_grad_(True) for n, p in lay.named_params()}
    xr = x.clone().requires_grad_(True)
    w = P["mu_w"] + P["sigma_w"] * (lay.f_in[:, None] * lay.f_out[None])
    b = P["mu_b"] + P["sigma_b"] * lay.f_out
    ref = xr @ w + b
    ref.backward(dy)
    y = lay.forward(x)
    dx = lay.vjp(dy)
    assert torch.allclose(y, ref, atol=1e-5) and torch.allclose(dx, xr.grad, atol=1e-5)
    for n, p in lay.named_params():
        assert torch.allclose(p.grad, P[n].grad, atol=1e-5), n
    lay.eval()
    assert torch.allclose(lay.forward(x), x @ P["mu_w"].detach() + P["mu_b"].detach(), atol=1e-5)   # eval = the mean layer
    f0 = lay.f_out.clone()
    nn.reset_noise(nn.Sequential(lay), g)
    assert not torch.equal(f0, lay.f_out)


def test_block_linear_is_an_ensemble_of_independent_maps():
    from noeira_b200 import nn
    nn.manual_seed(0)
    lay = nn.BlockLinear(4, 3, blocks=5, act="tanh")
    g = torch.Generator().manual_seed(2)
    x = torch.randn(6, 5, 4, generator=g)
    dy = torch.randn(6, 5, 3, generator=g)
    W = lay.weight.data.clone().reshape(5, 4, 3).requires_grad_(True)
    b = lay.bias.data.clone().reshape(5, 3).requires_grad_(True)
    xr = x.clone().requires_grad_(True)
    ref = torch.tanh(torch.einsum("bki,kio->bko", xr, W) + b)
    ref.backward(dy)
    y = lay.forward(x)
    dx = lay.vjp(dy)
    assert torch.allclose(y, ref, atol=1e-6) and torch.allclose(dx, xr.grad, atol=1e-6)
    assert torch.allclose(lay.weight.grad.reshape(5, 4, 3), W.grad, atol=1e-6) and torch.allclose(lay.bias.grad.reshape(5, 3), b.grad, atol=1e-6)
    shared = lay.forward(x[:, 0])                                 # one input for every member
    assert torch.allclose(shared[:, 3], torch.tanh(x[:, 0] @ W[3].detach() + b[3].detach()), atol=1e-6)
    assert lay.vjp(dy).shape == (6, 4)


def test_n_step_collector_matches_direct_sums():
    from noeira_b200.agents.rainbow import NStepCollector
    n, gamma, E, T = 3, 0.9, 2, 9
    g = torch.Generator().manual_seed(0)
    obs = torch.arange(T + 1).float()[:, None, None].expand(T + 1, E, 1) + torch.tensor([0.0, 100.0])[None, :, None]
    rew = torch.rand(T, E, generator=g)
    done = torch.zeros(T, E)
    done[4, 0] = 1                                                 # env 0: episode ends after step 4
    done[8, 1] = 1
    col = NStepCollector(n, gamma, E, 1)
    got = []
    for t in range(T):
        s0, a0, R, sp, tm, k = col.push(obs[t], torch.full((E,), t), rew[t], obs[t + 1], done[t], done[t])
        got += [(float(s0[i]), int(a0[i]), float(R[i]), float(sp[i]), float(tm[i]), int(k[i])) for i in range(s0.shape[0])]
    exp = []
    for e in range(E):
        for t in range(T):
            m, R = 0, 0.0
            while m < n and t + m < T:
                R += gamma ** m * float(rew[t + m, e])
                m += 1
                if done[t + m - 1, e]:
                    break
            if m == n or done[t + m - 1, e]:
                exp.append((float(obs[t, e]), t, R, float(obs[t + m, e]), float(done[t + m - 1, e]), m))
    key = lambda r: (r[0], r[1])
    got, exp = sorted(got, key=key), sorted(exp, key=key)
    assert len(got) == len(exp)
    for a, b in zip(got, exp):
        assert a[:2] == b[:2] and abs(a[2] - b[2]) < 1e-5 and a[3:] == b[3:], (a, b)


def test_rainbow_gradient_and_cartpole():
    from noeira_b200.agents.rainbow import RainbowConfig, RainbowTrainer, run_rainbow
    cfg = RainbowConfig(hidden=64, n_atoms=21, v_min=0.0, v_max=60.0, lr=1e-3, batch=64, n_step=3, target_every=100,
                        gamma=0.97, seed=0)
    tr = RainbowTrainer(cfg)
    names = [n for n, _ in tr.q.named_params()]
    assert any(n.endswith("value.sigma_w") for n in names) and any(n.endswith("advantage.mu_b") for n in names)
    # priorities are per-sample cross entropies; the weighted loss is their weighted mean
    g = torch.Generator().manual_seed(0)
    s, sp = torch.randn(8, 4, generator=g), torch.randn(8, 4, generator=g)
    a, r, d = torch.randint(0, 2, (8,), generator=g), torch.rand(8, generator=g), torch.zeros(8)
    w = torch.rand(8, generator=g)
    out = tr.update(s, a, r, sp, d, n_step=torch.tensor([1, 2, 3, 3, 3, 1, 2, 3]), weights=w)
    assert out["priorities"].shape == (8,) and abs(float(out["loss"]) - float((w * out["priorities"]).mean())) < 1e-6
    env = _DiscreteCartPole(8, seed=0)
    rets = run_rainbow(env, tr, total_steps=16_000, learning_starts=400)
    assert len(rets) > 20
    first, last = sum(rets[:20]) / 20, sum(rets[-20:]) / 20
    assert last > 1.5 * first and last > 40, (first, last)
