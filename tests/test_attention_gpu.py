"""Flash attention (tcgen05) against an fp32 PyTorch reference of the same masked softmax-attention."""
import pytest
import torch

pytestmark = pytest.mark.gpu

CASES = [
    # B, Sq, Sk, Hq, Hkv, D, mask, frame
    (2, 128, 128, 2, 2, 64, None, 0),
    (1, 256, 256, 4, 4, 64, "causal", 0),
    (2, 300, 300, 3, 1, 64, "causal", 0),
    (1, 100, 602, 8, 8, 64, None, 0),
    (2, 384, 384, 4, 2, 128, None, 0),
    (1, 512, 512, 4, 1, 128, "block_causal", 64),
    (1, 1024, 1024, 2, 2, 64, "block_causal", 257),
    (2, 50, 243, 15, 5, 64, None, 0),
]


@pytest.fixture(params=[1, 2], ids=["one_tile", "two_tile"])
def fwd_mode(request):
    """Runs a forward test once per forward kernel (one / two query tiles per CTA)."""
    from noeira_b200.ops.attention import set_forward_mode
    old = set_forward_mode(request.param)
    yield request.param
    set_forward_mode(old)


@pytest.mark.parametrize("B,Sq,Sk,Hq,Hkv,D,mask,frame", CASES + [(1, 1000, 1000, 2, 1, 128, "causal", 0),
                                                                  (1, 640, 900, 2, 2, 64, None, 0)])
def test_flash_forward(B, Sq, Sk, Hq, Hkv, D, mask, frame, fwd_mode):
    from noeira_b200.ops import check_status
    from noeira_b200.ops.attention import attention_reference, flash_attention_forward
    torch.manual_seed(0)
    q = torch.randn(B, Sq, Hq, D, device="cuda").bfloat16()
    k = torch.randn(B, Sk, Hkv, D, device="cuda").bfloat16()
    v = torch.randn(B, Sk, Hkv, D, device="cuda").bfloat16()
    o, lse = flash_attention_forward(q, k, v, mask=mask, frame=frame)
    torch.cuda.synchronize()
    check_status()
    ro, rl = attention_reference(q, k, v, mask=mask, frame=frame)
    assert (o.float() - ro).abs().max().item() < 3e-2, (o.float() - ro).abs().max().item()
    assert (lse - rl).abs().max().item() < 2e-2


def test_flash_forward_key_padding_and_bias_and_packed_qkv(fwd_mode):
    from noeira_b200.ops import check_status
    from noeira_b200.ops.attention import attention_reference, flash_attention_forward
    torch.manual_seed(1)
    B, S, H, D = 2, 200, 4, 64
    qkv = torch.randn(B, S, 3, H, D, device="cuda").bfloat16()
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    valid = torch.ones(B, S, dtype=torch.bool, device="cuda")
    valid[0, 150:] = False
    valid[1, 17:40] = False
    bias = torch.randn(S, S, device="cuda") * 0.5
    bias[:, 5] = float("-inf")
    o, lse = flash_attention_forward(q, k, v, key_valid=valid, bias=bias)
    torch.cuda.synchronize()
    check_status()
    ro, rl = attention_reference(q, k, v, key_valid=valid, bias=bias)
    assert (o.float() - ro).abs().max().item() < 3e-2
    assert (lse - rl).abs().max().item() < 2e-2


BWD_CASES = [
    (2, 128, 128, 2, 2, 64, None, 0),
    (1, 300, 300, 4, 2, 64, "causal", 0),
    (2, 100, 260, 4, 4, 64, None, 0),
    (1, 384, 384, 4, 1, 128, "block_causal", 96),
    (2, 256, 256, 2, 2, 128, None, 0),
]


@pytest.fixture(params=[0, 1], ids=["gen2", "gen1"])
def bwd_mode(request):
    from noeira_b200.ops.attention import set_backward_mode
    old = set_backward_mode(request.param)
    yield request.param
    set_backward_mode(old)


@pytest.mark.parametrize("B,Sq,Sk,Hq,Hkv,D,mask,frame", BWD_CASES + [(1, 1000, 1000, 2, 1, 128, "causal", 0),
                                                                      (1, 640, 900, 4, 2, 64, None, 0),
                                                                      (1, 1024, 1024, 2, 2, 128, "block_causal", 256)])
def test_flash_backward(B, Sq, Sk, Hq, Hkv, D, mask, frame, bwd_mode):
    from noeira_b200.ops import check_status
    from noeira_b200.ops.attention import attention_reference, flash_attention_backward, flash_attention_forward
    torch.manual_seed(0)
    q = torch.randn(B, Sq, Hq, D, device="cuda").bfloat16()
    k = torch.randn(B, Sk, Hkv, D, device="cuda").bfloat16()
    v = torch.randn(B, Sk, Hkv, D, device="cuda").bfloat16()
    do = (torch.randn(B, Sq, Hq, D, device="cuda") * 0.5).bfloat16()
    o, lse = flash_attention_forward(q, k, v, mask=mask, frame=frame)
    dq, dk, dv = flash_attention_backward(q, k, v, o, lse, do, mask=mask, frame=frame)
    torch.cuda.synchronize()
    check_status()
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    ro, _ = attention_reference(qf, kf, vf, mask=mask, frame=frame)
    ro.backward(do.float())
    for name, g, r in (("dq", dq, qf.grad), ("dk", dk, kf.grad), ("dv", dv, vf.grad)):
        err = (g.float() - r).abs().max().item()
        assert err < 4e-2 * max(1.0, r.abs().max().item()), (name, err, r.abs().max().item())
