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


@pytest.mark.parametrize("M", [128, 1000, 4096])
def test_fused_mlp_group_forward_backward_matches_layers(M):
    """Two networks (actor 17→6, critic 17→1) through the grouped forward, the fused data-gradient chain and the
    per-layer parameter-gradient branches, against the layer-by-layer explicit backward with the same weights."""
    from noeira_b200 import nn
    from noeira_b200.ops import check_status
    from noeira_b200.ops.mlp import Mlp3Pass, mlp3_backward_group, mlp3_forward_group, mlp3_param_grads
    from noeira_b200.ops.streams import Branch
    outs = (6, 1)
    mk = lambda o: nn.Sequential(nn.Linear(17, 256, act="tanh", need_input_grad=False), nn.Linear(256, 256, act="tanh"),
                                 nn.Linear(256, o, out_fp32=True)).to("cuda")
    nn.manual_seed(4)
    fused = [mk(o) for o in outs]
    nn.manual_seed(4)
    plain = [mk(o) for o in outs]
    x = torch.zeros(M, 24, device="cuda", dtype=torch.bfloat16)
    x[:, :17] = torch.randn(M, 17, device="cuda")
    dys = []
    for o in outs:
        d = torch.zeros(M, 8, device="cuda", dtype=torch.bfloat16)
        d[:, :o] = torch.randn(M, o, device="cuda") * 0.1
        d[:, o:] = 7.0                      # padding columns must be ignored
        dys.append(d)
    passes = [Mlp3Pass(*net.mods, M, x.device) for net in fused]
    ys = mlp3_forward_group(passes, [x, x])
    mlp3_backward_group(passes, [x, x], dys)
    branches = [[Branch(torch.cuda.Stream(), 1 + 3 * i + j) for j in range(3)] for i in range(2)]
    for p, d, br in zip(passes, dys, branches):
        mlp3_param_grads(p, x, d, br)
    for br in branches:
        for b in br:
            b.join()
    for net, d, o in zip(plain, dys, outs):
        net.forward(x[:, :17])
        net.vjp(d[:, :o])
    torch.cuda.synchronize()
    check_status()
    for p, net, y in zip(passes, plain, ys):
        ref = net.mods[2]._saved.float() if net.mods[2]._saved is not None else None
        assert (p.h1.float() - net.mods[0]._saved.float()).abs().max().item() < 2e-2
        assert (p.h2.float() - net.mods[1]._saved.float()).abs().max().item() < 3e-2
        if ref is not None:
            assert (y - ref[:, : y.shape[1]]).abs().max().item() < 3e-2 * max(1.0, ref.abs().max().item())
    for fn, pn in zip(fused, plain):
        for (n, pa), (_, pb) in zip(fn.named_params(), pn.named_params()):
            cos = torch.nn.functional.cosine_similarity(pa.grad.flatten(), pb.grad.flatten(), dim=0).item()
            rel = (pa.grad - pb.grad).abs().max().item() / max(pb.grad.abs().max().item(), 1e-6)
            assert cos > 0.999 and rel < 3e-2, (n, cos, rel)
