"""Fused three-layer MLP forward against the layer-by-layer path (same weights), including the backward caches."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("in_dim,out_dim,act,M", [(17, 6, "tanh", 4096), (17, 1, "tanh", 1000), (23, 1, "relu", 300), (64, 16, "tanh", 128)])
def test_fused_mlp_matches_layers(in_dim, out_dim, act, M):
    from noeira_b200 import nn
    from noeira_b200.ops import check_status
    from noeira_b200.ops.mlp import fusable, mlp3_forward
    nn.manual_seed(2)
    mk = lambda: nn.Sequential(nn.Linear(in_dim, 256, act=act, need_input_grad=False), nn.Linear(256, 256, act=act),
                               nn.Linear(256, out_dim, out_fp32=True)).to("cuda")
    a = mk()
    nn.manual_seed(2)
    b = mk()
    for net in (a, b):
        for i, m in enumerate(net.mods):
            m.bias.data.copy_(torch.linspace(-0.2, 0.2, m.bias.data.numel(), device="cuda") * (i + 1))
            m.bias.version += 1
    assert fusable(*a.mods)
    pad = (in_dim + 7) // 8 * 8
    x = torch.zeros(M, pad, device="cuda", dtype=torch.bfloat16)
    x[:, :in_dim] = torch.randn(M, in_dim, device="cuda")
    ya = mlp3_forward(x, *a.mods, save=True)
    yb = b.forward(x[:, :in_dim])
    torch.cuda.synchronize()
    check_status()
    err = (ya - yb.float()).abs().max().item()
    assert err < 2e-2 * max(1.0, yb.float().abs().max().item()), err
    assert (a.mods[0]._saved.float() - b.mods[0]._saved.float()).abs().max().item() < 2e-2
    assert (a.mods[1]._saved.float() - b.mods[1]._saved.float()).abs().max().item() < 3e-2
    g = (torch.randn(M, out_dim, device="cuda") * 0.1).bfloat16()
    a.vjp(g)
    b.vjp(g)
    torch.cuda.synchronize()
    for (n, pa), (_, pb) in zip(a.named_params(), b.named_params()):
        cos = torch.nn.functional.cosine_similarity(pa.grad.flatten(), pb.grad.flatten(), dim=0).item()
        assert cos > 0.995, (n, cos)


def test_ppo_fused_and_unfused_agree():
    from noeira_b200.agents.ppo import PPOConfig, PPOTrainer
    from noeira_b200.envs import PlanarChainEnv
    out = []
    for fused in (True, False):
        env = PlanarChainEnv(8192, seed=5)
        tr = PPOTrainer(env, PPOConfig(n_envs=8192, rollout_len=2, n_epochs=1, n_minibatches=2, fused_mlp=fused, use_cuda_graphs=False))
        assert bool(tr._fused.get(id(tr.actor))) == fused
        tr._rollout()
        torch.cuda.synchronize()
        out.append((tr.act_buf.clone(), tr.logp_buf.clone(), tr.rew_buf.clone()))
    assert (out[0][0][0] - out[1][0][0]).abs().max().item() < 5e-2     # first step: same noise stream, means equal to bf16 rounding
    assert (out[0][1][0] - out[1][1][0]).abs().max().item() < 0.2
