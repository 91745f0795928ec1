import torch

from noeira_b200 import nn


def test_q4_0_roundtrip_error_bound():
    torch.manual_seed(0)
    w = torch.randn(64, 128)
    codes, scales = nn.quantize_q4_0(w)
    assert codes.shape == (64, 64) and scales.shape == (64, 4) and scales.dtype == torch.float16
    back = nn.dequantize_q4_0(codes, scales)
    blk = w.reshape(64, 4, 32)
    step = blk.abs().amax(-1, keepdim=True) / 8
    err = (back.reshape(64, 4, 32) - blk).abs()
    assert (err <= step * 1.01 + 1e-3).all() and (err <= step * 0.51 + 1e-3).float().mean() > 0.97   # only the clamped far side exceeds half a step
    # the extreme of every block is reproduced (it defines the scale)
    i = blk.abs().argmax(-1, keepdim=True)
    assert torch.allclose(back.reshape(64, 4, 32).gather(-1, i), blk.gather(-1, i), rtol=2e-3, atol=1e-3)


def test_lora_gradients_freeze_and_merge():
    nn.manual_seed(0)
    base = nn.Linear(12, 16)
    lora = nn.LoRALinear(base, rank=8, alpha=16)
    assert [n for n, _ in lora.named_params()] == ["base_layer.weight", "base_layer.bias", "lora_A.weight", "lora_B.weight"]
    assert base.weight.frozen and not lora.lora_a.weight.frozen
    lora.lora_b.weight.data.normal_(0, 0.3)
    lora.lora_b.weight.version += 1
    x, w = torch.randn(5, 12), torch.randn(5, 16)
    lora.zero_grad()
    y = lora.forward(x)
    dx = lora.vjp(w)
    A, B = lora.lora_a.weight.data.clone().requires_grad_(True), lora.lora_b.weight.data.clone().requires_grad_(True)
    xr = x.clone().requires_grad_(True)
    yr = xr @ base.weight.data + base.bias.data + 2.0 * (xr @ A) @ B
    assert torch.allclose(y, yr.detach(), atol=1e-5)
    (yr * w).sum().backward()
    assert torch.allclose(lora.lora_a.weight.grad, A.grad, atol=1e-5) and torch.allclose(lora.lora_b.weight.grad, B.grad, atol=1e-5)
    assert torch.allclose(dx, xr.grad, atol=1e-5)
    assert float(base.weight.grad.abs().sum()) == 0.0
    lora.merge()
    assert torch.allclose(lora.forward(x), yr.detach(), atol=1e-5)
    assert nn.freeze_params(lora, lambda n, p: n.startswith("lora_")) == 2


def test_qlinear_and_qlora_cpu():
    nn.manual_seed(1)
    lin = nn.Linear(16, 32, act="relu")
    q = nn.QLinear(lin)
    x = torch.randn(7, 16)
    ref = torch.relu(x @ nn.dequantize_q4_0(q.codes.data, q.scales.data) + lin.bias.data)
    assert torch.allclose(q.forward(x), ref, atol=1e-5)
    assert (q.forward(x) - lin.forward(x)).abs().max() < 0.5
    g = torch.randn(7, 32)
    dx = q.vjp(g)
    assert torch.allclose(dx, (g * (ref > 0)) @ nn.dequantize_q4_0(q.codes.data, q.scales.data).t(), atol=1e-5)
    ql = nn.QLoRALinear(nn.Linear(16, 32), rank=8)
    trainable = [n for n, p in ql.named_params() if not p.frozen]
    assert trainable == ["lora_A.weight", "lora_B.weight"]
    assert [n for n, _ in ql.named_states()] == ["base_layer.qweight", "base_layer.scales"]
