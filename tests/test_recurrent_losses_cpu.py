import torch

from noeira_b200 import nn
from noeira_b200.nn import losses


def _copy_gru(cell, ref):
    H = cell.hidden
    with torch.no_grad():
        ref.weight_ih.copy_(cell.ih.weight.data.t())
        ref.weight_hh.copy_(cell.hh.weight.data.t())
        ref.bias_ih.copy_(cell.ih.bias.data)
        ref.bias_hh.copy_(cell.hh.bias.data)


def test_gru_cell_matches_torch():
    nn.manual_seed(0)
    cell = nn.GRUCell(5, 8)
    ref = torch.nn.GRUCell(5, 8)
    _copy_gru(cell, ref)
    x, h = torch.randn(4, 5), torch.randn(4, 8)
    xr, hr = x.clone().requires_grad_(True), h.clone().requires_grad_(True)
    out = cell.forward(x, h)
    outr = ref(xr, hr)
    assert torch.allclose(out, outr.detach(), atol=1e-5)
    g = torch.randn(4, 8)
    cell.zero_grad()
    dx, dh = cell.vjp(g)
    (outr * g).sum().backward()
    assert torch.allclose(dx, xr.grad, atol=1e-5) and torch.allclose(dh, hr.grad, atol=1e-5)
    assert torch.allclose(cell.ih.weight.grad, ref.weight_ih.grad.t(), atol=1e-5)
    assert torch.allclose(cell.hh.bias.grad, ref.bias_hh.grad, atol=1e-5)


def test_lstm_seq_matches_torch():
    nn.manual_seed(1)
    seq = nn.LSTMSeq(6, 7)
    ref = torch.nn.LSTM(6, 7, batch_first=True)
    with torch.no_grad():
        ref.weight_ih_l0.copy_(seq.cell.ih.weight.data.t())
        ref.weight_hh_l0.copy_(seq.cell.hh.weight.data.t())
        ref.bias_ih_l0.copy_(seq.cell.ih.bias.data)
        ref.bias_hh_l0.zero_()
    x = torch.randn(3, 5, 6)
    xr = x.clone().requires_grad_(True)
    out = seq.forward(x)
    outr, _ = ref(xr)
    assert torch.allclose(out, outr.detach(), atol=1e-5)
    g = torch.randn(3, 5, 7)
    seq.zero_grad()
    dx = seq.vjp(g)
    (outr * g).sum().backward()
    assert torch.allclose(dx, xr.grad, atol=1e-5)
    assert torch.allclose(seq.cell.ih.weight.grad, ref.weight_ih_l0.grad.t(), atol=1e-4)
    assert torch.allclose(seq.cell.hh.weight.grad, ref.weight_hh_l0.grad.t(), atol=1e-4)
    assert [n for n, _ in seq.named_params()] == ["cell.ih.weight", "cell.ih.bias", "cell.hh.weight"]


def test_losses_gradients_match_autograd():
    torch.manual_seed(0)
    mu, ls, t = torch.randn(6, 3, requires_grad=True), (torch.randn(6, 3) * 0.5).requires_grad_(True), torch.randn(6, 3)
    loss, dmu, dls = losses.gaussian_nll(mu, ls, t)
    ref = torch.nn.functional.gaussian_nll_loss(mu, t, torch.exp(2 * ls), full=True)
    assert torch.allclose(loss, ref.detach(), atol=1e-5)
    ref.backward()
    assert torch.allclose(dmu, mu.grad, atol=1e-6) and torch.allclose(dls, ls.grad, atol=1e-6)
    x, y = torch.randn(10, requires_grad=True), (torch.rand(10) > 0.5).float()
    l, dx = losses.bce_with_logits(x, y)
    r = torch.nn.functional.binary_cross_entropy_with_logits(x, y)
    r.backward()
    assert torch.allclose(l, r.detach(), atol=1e-6) and torch.allclose(dx, x.grad, atol=1e-6)
    bins = torch.linspace(-5, 5, 41)
    tgt = torch.tensor([0.0, 3.7, -120.0, 0.26])
    enc = losses.two_hot(losses.symlog(tgt), bins)
    assert torch.allclose(enc.sum(-1), torch.ones(4)) and ((enc > 0).sum(-1) <= 2).all()
    assert torch.allclose((enc * bins).sum(-1), losses.symlog(tgt).clamp(-5, 5), atol=1e-5)
    lg = torch.randn(4, 41, requires_grad=True)
    l2, dlg = losses.two_hot_loss(lg, tgt, bins)
    (-(enc * torch.log_softmax(lg, -1)).sum(-1).mean()).backward()
    assert torch.allclose(dlg, lg.grad, atol=1e-6)
    sharp = torch.log(enc + 1e-9)
    assert torch.allclose(losses.two_hot_decode(sharp, bins)[[0, 1, 3]], tgt[[0, 1, 3]], atol=1e-3)
    p, q, m = torch.randn(3, 5, 2), torch.randn(3, 5, 2), torch.tensor([[1, 1, 1, 0, 0], [1, 1, 1, 1, 1], [0, 0, 0, 0, 0]])
    per, g = losses.l1_masked_per_sample(p, q, m)
    assert abs(per[0].item() - (p - q)[0, :3].abs().mean().item()) < 1e-6 and per[2] == 0 and g[0, 3:].abs().sum() == 0
