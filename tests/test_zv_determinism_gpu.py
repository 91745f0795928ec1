"""Run-twice bit equality: the same inputs through the same kernel give the same bits (no atomics in any reduction of
these paths; the one documented exception is the embedding weight gradient, which is not covered here)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("D,mask,frame", [(64, "causal", 0), (128, "block_causal", 64), (64, None, 0)])
def test_flash_attention_forward_backward_repeat_bit_exact(D, mask, frame):
    from noeira_b200.ops import check_status
    from noeira_b200.ops.attention import flash_attention_backward, flash_attention_forward
    torch.manual_seed(0)
    B, S, Hq, Hkv = 2, 384, 4, 2
    q = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
    k = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    v = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    do = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
    outs = []
    for _ in range(2):
        o, lse = flash_attention_forward(q, k, v, mask=mask, frame=frame)
        dq, dk, dv = flash_attention_backward(q, k, v, o, lse, do, mask=mask, frame=frame)
        torch.cuda.synchronize()
        outs.append((o.clone(), lse.clone(), dq.clone(), dk.clone(), dv.clone()))
    check_status()
    for a, b in zip(*outs):
        assert torch.equal(a, b)


@pytest.mark.parametrize("ic,oc,k,s,p,hw", [(64, 64, 3, 1, 1, 32), (8, 64, 7, 2, 3, 64), (64, 128, 3, 2, 1, 32)])
def test_conv_forward_backward_repeat_bit_exact(ic, oc, k, s, p, hw):
    from noeira_b200 import nn
    from noeira_b200.ops import check_status
    nn.manual_seed(0)
    conv = nn.Conv2D(ic, oc, k, stride=s, pad=p).to("cuda")
    x = torch.randn(4, hw, hw, conv.icp, device="cuda").bfloat16()
    outs = []
    for _ in range(2):
        conv.zero_grad()
        y = conv.forward(x)
        dx = conv.vjp(torch.ones_like(y) * 0.01)
        torch.cuda.synchronize()
        outs.append((y.clone(), dx.clone() if dx is not None else y.clone(), conv.weight.grad.clone(), conv.bias.grad.clone()))
    check_status()
    for a, b in zip(*outs):
        assert torch.equal(a, b)


def test_tp_kernels_repeat_bit_exact_single_rank():
    from noeira_b200.ops import check_status
    from noeira_b200.parallel.tp import TPLinearContext
    g = torch.Generator(device="cuda").manual_seed(0)
    ms, k, n = 256, 512, 384
    ag, rs = TPLinearContext(1, 0, ms, k, n, "ag"), TPLinearContext(1, 0, ms, k, n, "rs")
    w = (torch.randn(k, n, device="cuda", generator=g) * 0.05).bfloat16()
    x = torch.randn(ms, k, device="cuda", generator=g).bfloat16()
    res = torch.randn(ms, n, device="cuda", generator=g).bfloat16()
    ag.x_shard.copy_(x)
    outs = []
    for _ in range(2):
        y = ag.ag_gemm(w, True, act="gelu")
        z = rs.gemm_rs(x, w, True, residual=res)
        torch.cuda.synchronize()
        outs.append((y.clone(), z.clone()))
    check_status()
    for a, b in zip(*outs):
        assert torch.equal(a, b)
