"""The eager tape: every operation against central differences, broadcasting, the module bridge against the module's own
backward, parameters through the arena optimizer, reset / no_grad, and a small training run."""
import pytest
import torch

from noeira_b200.experimental.functional import F, Tape, TapeAdam


def _check(fn, *shapes, seed=0, tol=1e-6, positive=False):
    """fn(tape, *leaves) → scalar FTensor; compares every leaf gradient with central differences in float64."""
    g = torch.Generator().manual_seed(seed)
    vals = [torch.randn(*s, generator=g, dtype=torch.float64) for s in shapes]
    if positive:
        vals = [v.abs() + 0.5 for v in vals]
    tape = Tape(dtype=torch.float64)
    leaves = [tape.input(v.clone()) for v in vals]
    out = fn(tape, *leaves)
    out.backward()
    for k, v in enumerate(vals):
        num = torch.zeros_like(v)
        flat = v.reshape(-1)
        for i in range(flat.numel()):
            old = float(flat[i])
            res = []
            for e in (1e-5, -1e-5):
                flat[i] = old + e
                t2 = Tape(dtype=torch.float64)
                with t2.no_grad():
                    res.append(fn(t2, *[t2.constant(x.clone()) for x in vals]).item())
            flat[i] = old
            num.reshape(-1)[i] = (res[0] - res[1]) / 2e-5
        got = leaves[k].grad
        assert got is not None and got.shape == v.shape
        assert (got - num).abs().max() < tol * max(1.0, float(num.abs().max())), (k, got, num)


def test_arithmetic_and_broadcasting_gradients():
    _check(lambda t, a, b: ((a + b) * (a - b) / (b * b + 2.0)).sum(), (3, 4), (1, 4))
    _check(lambda t, a, b: (a * b).mean() + (-a).sum() * 0.1 + (2.0 - b).sum() + (1.0 / (b * b + 1.0)).sum(), (2, 3, 4), (4,))
    _check(lambda t, a: (a ** 3.0).sum() + (a ** 2.0).mean(0).sum(), (3, 5))


def test_matrix_and_shape_operations():
    _check(lambda t, a, b: ((a @ b).T() @ a).sum(), (4, 3), (3, 4))
    _check(lambda t, a, b: (a @ b).sum(1).max(0).sum(), (2, 4, 3), (2, 3, 5))            # batched matmul
    _check(lambda t, a: (a.reshape(6, 4).permute(1, 0).narrow(0, 1, 2) ** 2.0).sum(), (2, 3, 4))
    _check(lambda t, a: (a.transpose(0, 2).sum((0, 1)) ** 2.0).sum() + a.max(1, keepdim=True).sum(), (2, 3, 4))
    _check(lambda t, a, b: (F.concat([a, b], 1) ** 2.0).sum() + F.gather(a, 1, torch.tensor([[0, 2], [1, 1], [2, 0]])).sum(), (3, 3), (3, 2))


def test_elementwise_functions_and_losses():
    _check(lambda t, a: (a.exp() + a.log() + a.sqrt()).sum(), (3, 4), positive=True)
    _check(lambda t, a: a.clamp(-0.5, 0.7).sum() + (a.tanh() * a.sigmoid()).sum() + a.gelu().sum() + a.silu().sum(), (4, 5))
    _check(lambda t, a: (a.softmax(-1) ** 2.0).sum() + (a.log_softmax(0) * 0.3).sum(), (3, 4))
    _check(lambda t, a: F.cross_entropy(a, torch.tensor([1, 0, 3])), (3, 4))
    _check(lambda t, a, g, b: (F.layer_norm(a, g, b) ** 2.0).sum(), (3, 6), (1, 6), (1, 6))
    for act in (None, "relu", "tanh", "gelu"):
        _check(lambda t, x, w, b: (F.linear(x, w, b, act) ** 2.0).sum(), (4, 3), (3, 5), (1, 5), seed=3)
    _check(lambda t, x, w: F.mse(F.linear(x, w), 0.5), (4, 3), (3, 2))


def test_a_broken_backward_is_caught():
    """The gradient check is not vacuous: a wrong derivative rule fails it."""
    from noeira_b200.experimental import functional as fn
    good = fn._BACKWARD["exp"]
    fn._BACKWARD["exp"] = lambda n: fn._acc(n.inputs[0], n.grad)
    try:
        with pytest.raises(AssertionError):
            _check(lambda t, a: a.exp().sum(), (2, 3))
    finally:
        fn._BACKWARD["exp"] = good


def test_module_bridge_matches_the_modules_own_backward():
    from noeira_b200 import nn
    torch.manual_seed(0)
    x = torch.randn(8, 16)

    def build():
        torch.manual_seed(1)
        return nn.Sequential(nn.Linear(16, 32, act="tanh"), nn.LayerNorm(32), nn.Linear(32, 4))

    ref = build()
    y = ref.forward(x)
    ref.vjp(2 * y / y.numel())
    tape = Tape()
    twin = build()
    for (_, p1), (_, p2) in zip(ref.named_params(), twin.named_params()):
        p2.data.copy_(p1.data)
    net = tape.module(twin, "net")
    xin = tape.input(x)
    loss = (net(xin) ** 2.0).mean()
    loss.backward()
    for (n1, p1), (n2, p2) in zip(ref.named_params(), tape.named_params()):
        assert n2 == "net." + n1 and torch.allclose(p1.grad, p2.grad, atol=1e-6), n1
    assert xin.grad.shape == x.shape and abs(loss.item() - float((y ** 2).mean())) < 1e-6
    # a module on a CONSTANT input is still recorded: its own parameters need the reverse pass
    tape.reset()
    tape.zero_grad()
    (net(tape.constant(x)) ** 2.0).mean().backward()
    for (n1, p1), (_, p2) in zip(ref.named_params(), tape.named_params()):
        assert torch.allclose(p1.grad, p2.grad, atol=1e-6), n1


def test_training_with_the_arena_optimizer_reset_and_no_grad():
    tape = Tape(seed=0)
    w1, b1 = tape.param(2, 32, name="w1"), tape.zeros(1, 32, name="b1")
    w2, b2 = tape.param(32, 1, "xavier", name="w2"), tape.zeros(1, 1, name="b2")
    assert [n for n, _ in tape.named_params()] == ["w1", "b1", "w2", "b2"]
    opt = TapeAdam(tape, lr=1e-2)
    g = torch.Generator().manual_seed(0)
    x = torch.rand(256, 2, generator=g) * 2 - 1
    y = torch.sin(3 * x[:, :1]) * x[:, 1:]
    first = None
    for step in range(300):
        tape.reset()
        loss = F.mse(F.linear(F.linear(tape.constant(x), w1, b1, "tanh"), w2, b2), y)
        loss.backward()
        opt.step()
        first = first if first is not None else loss.item()
    assert loss.item() < 0.25 * first
    n_nodes = len(tape)
    tape.reset()
    assert len(tape) == 0 and n_nodes == 5          # two fused linears, the difference, its square, the mean
    with tape.no_grad():
        out = F.linear(tape.constant(x), w1, b1, "tanh")
    assert len(tape) == 0 and out.shape == (256, 32)
    with pytest.raises(KeyError):
        tape.param(2, 2, name="w1")
    # the same seed gives the same initial values and the same dropout masks
    t2 = Tape(seed=0)
    assert torch.equal(t2.param(2, 32, name="w1").value, Tape(seed=0).param(2, 32, name="w1").value)
    a = F.dropout(Tape(seed=5).constant(torch.ones(4, 4)), 0.5).value
    b = F.dropout(Tape(seed=5).constant(torch.ones(4, 4)), 0.5).value
    assert torch.equal(a, b) and set(a.unique().tolist()) <= {0.0, 2.0}
