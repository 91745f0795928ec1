"""LoRA / Q4_0 layers and the GPT model on CUDA against the CPU oracle; graphed autoregressive training."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _cmp(a, b, tol, what=""):
    err = (a.float().cpu() - b.float().cpu()).abs().max().item()
    ref = b.float().abs().max().item()
    assert err <= tol * max(1.0, ref), (what, err, ref)


def test_qlinear_lora_gpu_match_cpu():
    from noeira_b200 import nn
    nn.manual_seed(5)
    lin = nn.Linear(64, 96, act="relu")
    qc = nn.QLinear(lin)
    nn.manual_seed(5)
    qg = nn.QLinear(nn.Linear(64, 96, act="relu")).to("cuda")
    w_cpu = nn.dequantize_q4_0(qc.codes.data, qc.scales.data)
    w_gpu = nn.dequantize_q4_0(qg.codes.data, qg.scales.data, torch.float32)
    assert torch.equal(w_cpu.bfloat16().float(), w_gpu.cpu())           # the kernel decodes every block exactly
    x = torch.randn(33, 64)
    _cmp(qg.forward(x.cuda().bfloat16()), qc.forward(x), 3e-2, "qlinear fwd")
    g = torch.randn(33, 96)
    qc.forward(x)
    dxg, dxc = qg.vjp(g.cuda().bfloat16()).float().cpu(), qc.vjp(g)
    # a few ReLU outputs within rounding of zero take the other branch in bf16: compare direction and norm
    assert torch.nn.functional.cosine_similarity(dxg.flatten(), dxc.flatten(), dim=0) > 0.99
    assert 0.95 < (dxg.norm() / dxc.norm()).item() < 1.05
    nn.manual_seed(6)
    lc = nn.LoRALinear(nn.Linear(64, 96), rank=8)
    nn.manual_seed(6)
    lg = nn.LoRALinear(nn.Linear(64, 96), rank=8)
    for m in (lc, lg):
        m.lora_b.weight.data.copy_(torch.linspace(-0.3, 0.3, 8 * 96).reshape(8, 96))
        m.lora_b.weight.version += 1
    lg.to("cuda")
    _cmp(lg.forward(x.cuda().bfloat16()), lc.forward(x), 3e-2, "lora fwd")
    lc.vjp(g)
    lg.vjp(g.cuda().bfloat16())
    torch.cuda.synchronize()
    _cmp(lg.lora_a.weight.grad, lc.lora_a.weight.grad, 5e-2, "dA")
    _cmp(lg.lora_b.weight.grad, lc.lora_b.weight.grad, 5e-2, "dB")
    assert float(lg.base.weight.grad.abs().sum()) == 0.0


def test_gpt_gpu_matches_cpu_and_trains():
    from noeira_b200 import nn
    from noeira_b200.models.gpt import GPT
    from noeira_b200.training import AutoregressiveTrainer
    for tie in (False, True):
        cpu = GPT(vocab=64, seq=32, dim=128, layers=2, heads=2, tie=tie, seed=3)
        gpu = GPT(vocab=64, seq=32, dim=128, layers=2, heads=2, tie=tie, seed=3).to("cuda")
        ids = torch.randint(0, 64, (4, 32))
        lc, lg = cpu.forward(ids), gpu.forward(ids.cuda())
        _cmp(lg, lc, 5e-2, "logits")
        tgt = torch.randint(0, 64, (4, 32))
        ac, ag = torch.zeros(1), torch.zeros(1, device="cuda")
        cpu.vjp(nn.cross_entropy(lc, tgt, ac))
        gpu.vjp(nn.cross_entropy(lg.contiguous(), tgt.cuda(), ag))
        torch.cuda.synchronize()
        assert abs(ac.item() - ag.item()) < 5e-2
        for (n, pc), (_, pg) in zip(cpu.named_params(), gpu.named_params()):
            c = torch.nn.functional.cosine_similarity(pc.grad.flatten(), pg.grad.cpu().flatten(), dim=0).item()
            assert pc.grad.abs().max() < 1e-7 or c > 0.97, (tie, n, c)
    toks = (torch.arange(6000) % 11).cuda()
    lm = GPT(vocab=16, seq=32, dim=128, layers=2, heads=2, seed=0).to("cuda")
    tr = AutoregressiveTrainer(lm, toks, batch=16, seq=32, lr=3e-3, warmup=5, total_steps=80, use_cuda_graph=True)
    tr.train_step()
    first = tr.mean_loss()
    for _ in range(79):
        tr.train_step()
    assert tr._graphed.graph is not None
    assert tr.mean_loss() / 79 < 0.5 * first
