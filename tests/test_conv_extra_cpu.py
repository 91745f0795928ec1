"""Transposed convolution, average pooling and nearest upsampling: explicit backward against autograd (CPU path)."""
import pytest
import torch


@pytest.mark.parametrize("k,stride,pad", [(4, 2, 1), (3, 1, 1), (2, 2, 0), (3, 2, 0)])
def test_conv_transpose_matches_torch(k, stride, pad):
    from noeira_b200 import nn
    nn.manual_seed(0)
    lay = nn.Conv2DTranspose(6, 5, k, stride=stride, pad=pad, relu=True)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(2, 5, 7, 6, generator=g)
    w = lay._w_torch().clone().requires_grad_(True)
    b = lay.bias.data.clone().requires_grad_(True)
    xr = x.clone().requires_grad_(True)
    ref = torch.relu(torch.nn.functional.conv_transpose2d(xr.permute(0, 3, 1, 2), w, b, stride, pad)).permute(0, 2, 3, 1)
    y = lay.forward(x)
    assert y.shape == (2, *lay.out_hw(5, 7), 5) and torch.allclose(y, ref, atol=1e-5)
    dy = torch.randn(y.shape, generator=g)
    ref.backward(dy)
    dx = lay.vjp(dy)
    assert torch.allclose(dx, xr.grad, atol=1e-4)
    gw = lay.weight.grad.view(k, k, lay.ocp, 6)[:, :, :5].permute(3, 2, 0, 1)
    assert torch.allclose(gw, w.grad, atol=1e-4) and torch.allclose(lay.bias.grad, b.grad, atol=1e-4)
    # files hold the torch layout
    f = lay.weight.file_view()
    assert f.shape == (6, 5, k, k) and torch.allclose(f, w.detach())
    lay2 = nn.Conv2DTranspose(6, 5, k, stride=stride, pad=pad)
    lay2.weight.load_file_(f.reshape(-1))
    assert torch.allclose(lay2._w_torch(), w.detach())


def test_avgpool_and_upsample_backward():
    from noeira_b200 import nn
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, 7, 6, 3, generator=g, requires_grad=True)
    pool, up = nn.AvgPool2D(2), nn.Upsample2D(3)
    ref = torch.nn.functional.avg_pool2d(x.permute(0, 3, 1, 2), 2).permute(0, 2, 3, 1)
    y = pool.forward(x.detach())
    assert torch.allclose(y, ref, atol=1e-6)
    dy = torch.randn(y.shape, generator=g)
    ref.backward(dy)
    assert torch.allclose(pool.vjp(dy), x.grad, atol=1e-6)
    x2 = torch.randn(2, 3, 4, 5, generator=g, requires_grad=True)
    ref = torch.nn.functional.interpolate(x2.permute(0, 3, 1, 2), scale_factor=3, mode="nearest").permute(0, 2, 3, 1)
    y = up.forward(x2.detach())
    assert torch.equal(y, ref)
    dy = torch.randn(y.shape, generator=g)
    ref.backward(dy)
    assert torch.allclose(up.vjp(dy), x2.grad, atol=1e-5)
