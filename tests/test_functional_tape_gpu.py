"""The eager tape on CUDA: the fused linear node and aligned matrix products run on the TF32 tensor-core GEMM and agree
with the CPU tape; a training run through the arena optimizer."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _net(tape, x, y, ps):
    from noeira_b200.experimental.functional import F
    w1, b1, w2, b2 = ps
    h = F.linear(tape.constant(x), w1, b1, "tanh")
    return F.mse(F.linear(h, w2, b2) + (h @ w2) * 0.5, y)


def test_cuda_tape_matches_the_cpu_tape_and_trains():
    from noeira_b200.experimental.functional import Tape, TapeAdam
    from noeira_b200.ops import check_status
    g = torch.Generator().manual_seed(0)
    x, y = torch.randn(256, 64, generator=g), torch.randn(256, 8, generator=g)
    tapes = {}
    for dev in ("cpu", "cuda"):
        t = Tape(device=dev, seed=1)
        ps = (t.param(64, 128, name="w1"), t.zeros(1, 128, name="b1"), t.param(128, 8, "xavier", name="w2"), t.zeros(1, 8, name="b2"))
        tapes[dev] = (t, ps)
    losses = {}
    for dev, (t, ps) in tapes.items():
        loss = _net(t, x.to(dev), y.to(dev), ps)
        loss.backward()
        losses[dev] = loss.item()
    torch.cuda.synchronize()
    check_status()
    assert abs(losses["cpu"] - losses["cuda"]) < 5e-3 * max(1.0, abs(losses["cpu"]))
    for (n, pc), (_, pg) in zip(tapes["cpu"][0].named_params(), tapes["cuda"][0].named_params()):
        scale = max(1e-3, float(pc.grad.abs().max()))
        assert (pc.grad - pg.grad.cpu()).abs().max() < 1e-2 * scale, n          # TF32 operands: 10-bit mantissa
    t, ps = tapes["cuda"]
    t.zero_grad()
    opt = TapeAdam(t, lr=3e-3)
    first = None
    for _ in range(200):
        t.reset()
        loss = _net(t, x.cuda(), y.cuda(), ps)
        loss.backward()
        opt.step()
        first = first if first is not None else loss.item()
    assert loss.item() < 0.7 * first


def test_module_node_on_cuda_runs_in_the_modules_activation_dtype():
    """An ``nn`` module inside a CUDA tape gets bf16 rows (what its kernels read) and hands fp32 back to the tape."""
    from noeira_b200 import nn
    from noeira_b200.experimental.functional import F, Tape
    g = torch.Generator().manual_seed(0)
    x, y = torch.randn(256, 64, generator=g), torch.randn(256, 8, generator=g)
    res = {}
    for dev in ("cpu", "cuda"):
        nn.manual_seed(3)
        t = Tape(device=dev, seed=2)
        net = t.module(nn.Sequential(nn.Linear(64, 64, act="tanh"), nn.LayerNorm(64)), "net")
        w = t.param(64, 8, "xavier", name="w")
        loss = F.mse(F.linear(net(t.constant(x.to(dev))), w), y.to(dev))
        loss.backward()
        res[dev] = (loss.item(), {n: p.grad.detach().float().cpu().clone() for n, p in t.named_params()})
    torch.cuda.synchronize()
    assert abs(res["cpu"][0] - res["cuda"][0]) < 0.03 * abs(res["cpu"][0])
    for n, gc in res["cpu"][1].items():
        gg = res["cuda"][1][n][tuple(slice(0, k) for k in gc.shape)]
        cos = float((gc * gg).sum() / (gc.norm() * gg.norm()).clamp_min(1e-30))
        assert cos > 0.99, (n, cos)
