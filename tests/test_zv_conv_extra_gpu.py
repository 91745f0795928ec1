"""Transposed convolution, average pooling, nearest upsampling on CUDA against the fp32 CPU path of the same modules."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("k,stride,pad", [(4, 2, 1), (3, 1, 1), (2, 2, 0)])
def test_conv_transpose_cuda_matches_cpu(k, stride, pad):
    from noeira_b200 import nn
    from noeira_b200.ops import check_status
    nn.manual_seed(0)
    # no fused ReLU here: an output within bf16 rounding of zero flips its mask between the two paths, and one flipped
    # element moves a weight-gradient entry by a whole |x · dy| term (the ReLU path is covered by the CPU test)
    cpu = nn.Conv2DTranspose(16, 12, k, stride=stride, pad=pad)
    nn.manual_seed(0)
    gpu = nn.Conv2DTranspose(16, 12, k, stride=stride, pad=pad).to("cuda")
    torch.manual_seed(1)
    x = torch.randn(3, 9, 10, 16)
    yc = cpu.forward(x)
    yg = gpu.forward(x.cuda().bfloat16())
    dy = torch.randn(yc.shape)
    dxc = cpu.vjp(dy)
    dxg = gpu.vjp(dy.cuda().bfloat16())
    torch.cuda.synchronize()
    check_status()
    assert (yg.float().cpu() - yc).abs().max().item() < 3e-2 * max(1.0, yc.abs().max().item())
    assert (dxg.float().cpu() - dxc).abs().mean().item() < 2e-2 * max(1.0, dxc.abs().mean().item())
    assert (gpu.weight.grad.cpu() - cpu.weight.grad).abs().max().item() < 5e-2 * max(1.0, cpu.weight.grad.abs().max().item())
    assert (gpu.bias.grad.cpu() - cpu.bias.grad).abs().max().item() < 5e-2 * max(1.0, cpu.bias.grad.abs().max().item())


def test_avgpool_upsample_cuda_match_cpu():
    from noeira_b200 import nn
    torch.manual_seed(0)
    x = torch.randn(2, 9, 8, 24)
    for mod_c, mod_g in ((nn.AvgPool2D(2), nn.AvgPool2D(2)), (nn.Upsample2D(2), nn.Upsample2D(2))):
        xb = x.bfloat16()
        yc = mod_c.forward(xb.float())
        yg = mod_g.forward(xb.cuda())
        assert (yg.float().cpu() - yc).abs().max().item() < 2e-2
        dy = torch.randn(yc.shape).bfloat16()
        dc = mod_c.vjp(dy.float())
        dg = mod_g.vjp(dy.cuda())
        assert (dg.float().cpu() - dc).abs().max().item() < 3e-2
