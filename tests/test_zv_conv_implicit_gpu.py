"""Implicit-GEMM convolution forward (patches read by the GEMM's TMA producer) against the patch-matrix path."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("ic,oc,k,pad,H,W", [(64, 64, 3, 1, 24, 32), (64, 128, 3, 1, 15, 48), (128, 64, 1, 0, 9, 80),
                                             (64, 96, 3, 0, 12, 18), (128, 128, 3, 1, 30, 160)])
def test_implicit_matches_patch_matrix(ic, oc, k, pad, H, W):
    from noeira_b200 import nn
    nn.manual_seed(3)
    a = nn.Conv2D(ic, oc, k, 1, pad, bias=True, relu=True).to("cuda")
    nn.manual_seed(3)
    b = nn.Conv2D(ic, oc, k, 1, pad, bias=True, relu=True).to("cuda")
    b.implicit_gemm = False
    a.force_implicit = True
    a.bias.data.normal_(0, 0.1)
    b.bias.data.copy_(a.bias.data)
    x = (torch.randn(3, H, W, ic, device="cuda") * 0.5).bfloat16()
    OW = W + 2 * pad - k + 1
    assert a._implicit_ok(ic, OW)
    ya, yb = a.forward(x), b.forward(x)
    torch.cuda.synchronize()
    from noeira_b200.ops import check_status
    check_status()
    assert a._col is None and b._col is not None
    # same K order; the patch-matrix GEMM may split K (another summation order), so allow bf16 rounding
    assert (ya.float() - yb.float()).abs().max().item() <= 2e-2 * max(1.0, yb.float().abs().max().item())
    assert (ya != yb).float().mean().item() < 0.05
    dy = (torch.randn_like(ya.float()) * 0.1).bfloat16()
    da, db = a.vjp(dy), b.vjp(dy)
    torch.cuda.synchronize()
    # the backward of both runs through the patch matrix; only ReLU masks of outputs that differ in sign can differ
    cos = lambda u, v: torch.nn.functional.cosine_similarity(u.float().flatten(), v.float().flatten(), dim=0).item()
    assert cos(da, db) > 0.999 and cos(a.weight.grad, b.weight.grad) > 0.999 and cos(a.bias.grad, b.bias.grad) > 0.999


@pytest.mark.parametrize("ic,oc,k,pad,H,W", [(64, 64, 3, 1, 24, 32), (128, 64, 3, 1, 15, 48), (64, 128, 3, 0, 20, 40)])
def test_implicit_input_gradient_matches_fp32_reference(ic, oc, k, pad, H, W):
    """dx of a stride-1 layer = a stride-1 convolution of dy with mirrored taps, run by the implicit-GEMM kernel."""
    from noeira_b200 import nn
    from noeira_b200.ops import check_status
    nn.manual_seed(7)
    c = nn.Conv2D(ic, oc, k, 1, pad, bias=False, relu=False).to("cuda")
    x = (torch.randn(2, H, W, ic, device="cuda") * 0.5).bfloat16()
    assert c._implicit_dgrad_ok(W)
    y = c.forward(x)
    dy = (torch.randn_like(y.float()) * 0.1).bfloat16()
    dx = c.vjp(dy)
    torch.cuda.synchronize()
    check_status()
    w = c.weight.shadow.float().view(k, k, ic, oc).permute(3, 2, 0, 1)
    ref = torch.nn.grad.conv2d_input((2, ic, H, W), w, dy.float().permute(0, 3, 1, 2), 1, pad).permute(0, 2, 3, 1)
    err = (dx.float() - ref).abs().max().item()
    assert err < 2e-2 * max(1.0, ref.abs().max().item()), err


@pytest.mark.parametrize("ic,oc,k,pad,H,W,B", [(64, 64, 3, 1, 24, 32, 3), (128, 96, 3, 1, 15, 48, 2), (64, 128, 3, 0, 12, 18, 4),
                                                (128, 64, 1, 0, 9, 80, 2), (64, 64, 3, 1, 30, 160, 8)])
def test_implicit_weight_gradient_matches_fp32_reference(ic, oc, k, pad, H, W, B):
    """dW from the NHWC input through the TMA producer (no patch matrix in forward or backward) against torch's fp32
    convolution weight gradient on the same bf16-rounded tensors; accumulation into an existing gradient; bit-repeatable."""
    from noeira_b200 import nn
    from noeira_b200.ops import check_status
    nn.manual_seed(4)
    lay = nn.Conv2D(ic, oc, k, 1, pad, bias=True).to("cuda")
    lay.implicit_wgrad = True
    OW = W + 2 * pad - k + 1
    assert lay._implicit_wgrad_ok(OW) and lay._implicit_ok(ic, OW)
    x = (torch.randn(B, H, W, ic, device="cuda") * 0.5).bfloat16()
    y = lay.forward(x)
    assert lay._col is None and lay._xin is not None                     # nothing but the input was kept
    dy = (torch.randn_like(y.float()) * 0.1).bfloat16()
    lay.weight.grad_storage.fill_(0.25)                                  # the kernel adds to what is there
    lay.vjp(dy)
    torch.cuda.synchronize()
    check_status()
    got = lay.weight.grad.clone() - 0.25
    w = lay.weight.data.view(k, k, ic, oc).permute(3, 2, 0, 1).float()
    ref = torch.nn.grad.conv2d_weight(x.float().permute(0, 3, 1, 2), w.shape, dy.float().permute(0, 3, 1, 2), 1, pad)
    ref = ref.permute(2, 3, 1, 0).reshape(k * k * ic, oc)
    scale = max(1.0, ref.abs().max().item())
    assert (got - ref).abs().max().item() < 2e-2 * scale, ((got - ref).abs().max().item(), scale)
    lay.weight.grad_storage.fill_(0.25)
    lay.forward(x)
    lay.vjp(dy)
    torch.cuda.synchronize()
    assert torch.equal(lay.weight.grad - 0.25, got)
