"""Transformer leaves on CUDA (our kernels, bf16) against the same modules on CPU (fp32 oracle)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _pair(factory):
    from noeira_b200 import nn
    nn.manual_seed(3)
    a = factory()
    nn.manual_seed(3)
    b = factory().to("cuda")
    return a, b


def _cmp(a, b, tol):
    err = (a.float().cpu() - b.float().cpu()).abs().max().item()
    ref = b.float().abs().max().item()
    assert err <= tol * max(1.0, ref), (err, ref)


@pytest.mark.parametrize("rms", [False, True])
def test_norm_fwd_bwd(rms):
    from noeira_b200 import nn
    cls = nn.RMSNorm if rms else nn.LayerNorm
    cpu, gpu = _pair(lambda: cls(960))
    cpu.gamma.set_(torch.randn(960) * 0.3 + 1)
    gpu.gamma.set_(cpu.gamma.data)
    x = torch.randn(3, 70, 960)
    dy = torch.randn(3, 70, 960)
    yc, yg = cpu.forward(x), gpu.forward(x.cuda().bfloat16())
    _cmp(yg, yc, 3e-2)
    dc, dg = cpu.vjp(dy), gpu.vjp(dy.cuda().bfloat16())
    torch.cuda.synchronize()
    _cmp(dg, dc, 4e-2)
    _cmp(gpu.gamma.grad, cpu.gamma.grad, 3e-2)
    if not rms:
        _cmp(gpu.beta.grad, cpu.beta.grad, 3e-2)


@pytest.mark.parametrize("cfg", [dict(norm="layer", ffn="gelu", mask=None, rope_theta=None, kv_heads=None, bias=True),
                                 dict(norm="rms", ffn="swiglu", mask="causal", rope_theta=1e4, kv_heads=2, bias=False),
                                 dict(norm="rms", ffn="swiglu", mask="block_causal", frame=40, rope_theta=None, kv_heads=1, bias=False)])
def test_transformer_block_matches_cpu(cfg):
    from noeira_b200 import nn
    from noeira_b200.ops import check_status
    cpu, gpu = _pair(lambda: nn.TransformerBlock(256, 4, 512, **cfg))
    x = torch.randn(2, 200, 256) * 0.5
    dy = torch.randn(2, 200, 256) * 0.1
    yc = cpu.forward(x)
    yg = gpu.forward(x.cuda().bfloat16())
    _cmp(yg, yc, 4e-2)
    dc = cpu.vjp(dy)
    dg = gpu.vjp(dy.cuda().bfloat16())
    torch.cuda.synchronize()
    check_status()
    _cmp(dg, dc, 5e-2)
    for (n, pc), (_, pg) in zip(cpu.named_params(), gpu.named_params()):
        err = (pg.grad.cpu() - pc.grad).abs().max().item()
        assert err <= 6e-2 * max(1.0, pc.grad.abs().max().item()), (n, err, pc.grad.abs().max().item())


def test_embedding_rope_losses():
    from noeira_b200 import nn
    cpu, gpu = _pair(lambda: nn.Embedding(1000, 64))
    idx = torch.randint(0, 1000, (4, 33))
    _cmp(gpu.forward(idx.cuda()), cpu.forward(idx), 1e-2)
    dy = torch.randn(4, 33, 64)
    cpu.vjp(dy)
    gpu.vjp(dy.cuda().bfloat16())
    _cmp(gpu.weight.grad, cpu.weight.grad, 3e-2)
    x = torch.randn(2, 50, 3, 64)
    xr = nn.rope_(x.clone(), 1e4)
    xg = nn.rope_(x.cuda().bfloat16(), 1e4)
    _cmp(xg, xr, 3e-2)
    _cmp(nn.rope_(xg.clone(), 1e4, backward=True), x, 5e-2)
    # losses
    pred, tgt = torch.randn(40, 32), torch.randn(40, 32)
    for l1 in (False, True):
        L = nn.MSELoss(l1=l1)
        acc_c, acc_g = torch.zeros(1), torch.zeros(1, device="cuda")
        gc = L(pred, tgt, acc_c, n_real=6)
        gg = L(pred.cuda().bfloat16(), tgt.cuda(), acc_g, n_real=6)
        assert abs(acc_c.item() - acc_g.item()) < 2e-2
        _cmp(gg, gc, 3e-2)
        acc_f = torch.zeros(1, device="cuda")
        gf = L(pred.cuda(), tgt.cuda(), acc_f, n_real=6)           # fp32 predictions are read as fp32
        assert abs(acc_c.item() - acc_f.item()) < 1e-4
        _cmp(gf, gc, 1e-2)
    logits = torch.randn(64, 500)
    tg = torch.randint(0, 500, (64,))
    acc_c, acc_g = torch.zeros(1), torch.zeros(1, device="cuda")
    gc = nn.cross_entropy(logits, tg, acc_c)
    gg = nn.cross_entropy(logits.cuda().bfloat16(), tg.cuda(), acc_g)
    assert abs(acc_c.item() - acc_g.item()) < 3e-2
    _cmp(gg, gc, 3e-2)
    t = torch.rand(9)
    _cmp(nn.sincos_embed(t.cuda(), 64), nn.sincos_embed(t, 64), 2e-2)
