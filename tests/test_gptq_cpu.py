"""GPTQ calibration of a Q4_0 linear layer: smaller output error than round-to-nearest on correlated inputs."""
import torch


def test_gptq_beats_round_to_nearest():
    from noeira_b200.nn.peft import dequantize_q4_0, gptq_quantize_q4_0, quantize_q4_0
    torch.manual_seed(0)
    IN, OUT, n = 96, 64, 2048
    mix = torch.randn(IN, IN) * 0.3 + torch.eye(IN)
    x = torch.randn(n, IN) @ mix                       # correlated input features
    w = torch.randn(IN, OUT) * 0.2
    rtn = dequantize_q4_0(*quantize_q4_0(w))
    codes, scales = gptq_quantize_q4_0(w, x)
    assert codes.shape == (IN, OUT // 2) and scales.shape == (IN, OUT // 32)
    gq = dequantize_q4_0(codes, scales)
    xt = torch.randn(512, IN) @ mix                    # held-out inputs of the same distribution
    e_rtn = (xt @ (w - rtn)).pow(2).mean().item()
    e_gptq = (xt @ (w - gq)).pow(2).mean().item()
    assert e_gptq < 0.6 * e_rtn, (e_gptq, e_rtn)
    # every weight stays on the 4-bit grid of its block
    blk = gq.reshape(IN, OUT // 32, 32) / scales.float().unsqueeze(-1)
    assert torch.allclose(blk, blk.round(), atol=1e-3) and blk.min() >= -8 and blk.max() <= 7


def test_qlinear_with_calibration_matches_the_dense_layer_more_closely():
    from noeira_b200 import nn
    from noeira_b200.nn.peft import QLinear
    nn.manual_seed(1)
    lin = nn.Linear(64, 64)
    torch.manual_seed(2)
    mix = torch.randn(64, 64) * 0.4 + torch.eye(64)
    x = torch.randn(1024, 64) @ mix
    ref = lin.forward(x)
    plain, cal = QLinear(lin), QLinear(lin, calibration=x)
    e_plain = (plain.forward(x) - ref).pow(2).mean().item()
    e_cal = (cal.forward(x) - ref).pow(2).mean().item()
    assert e_cal < e_plain
