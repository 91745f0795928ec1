"""ComputeGraph fan-out, schedulers, GPT / ViT explicit backward against finite differences, trainers (CPU oracle path)."""
import math

import torch

from noeira_b200 import nn


def _fd_check(loss_fn, params, eps=5e-3, n=6, tol=4e-2):
    base_grads = {name: p.grad.clone() for name, p in params}
    g = torch.Generator().manual_seed(0)
    for name, p in params:
        d, gr = p.data, base_grads[name]              # strided views of the padded storage: index, never flatten
        for _ in range(n):
            i = tuple(int(torch.randint(0, s, (1,), generator=g)) for s in d.shape)
            old = d[i].item()
            d[i] = old + eps
            p.version += 1
            lp = loss_fn()
            d[i] = old - eps
            p.version += 1
            lm = loss_fn()
            d[i] = old
            p.version += 1
            fd = (lp - lm) / (2 * eps)
            assert abs(fd - gr[i].item()) < tol * max(abs(fd), abs(gr[i].item())) + 3e-4, (name, fd, gr[i].item())


def test_compute_graph_fanout_and_names():
    nn.manual_seed(0)
    a, b, c = nn.Linear(5, 7, act="tanh"), nn.Linear(7, 3), nn.Linear(7, 3)
    add = nn.ExternalNode("sum", lambda u, v: u + v, lambda g, u, v: (g, g), ["b", "c"])
    G = nn.ComputeGraph([nn.InputSlot("x"), nn.Node("a", a, ["x"]), nn.Node("b", b, ["a"]), nn.Node("c", c, ["a"]), add])
    assert [n for n, _ in G.named_params()] == ["a.weight", "a.bias", "b.weight", "b.bias", "c.weight", "c.bias"]
    x = torch.randn(4, 5)
    w = torch.randn(4, 3)

    def loss():
        return float((G.forward(x) * w).sum())
    G.zero_grad()
    G.forward(x)
    gx = G.vjp(w)["x"]
    _fd_check(loss, list(G.named_params()))
    xr = x.clone().requires_grad_(True)
    h = torch.tanh(xr @ a.weight.data + a.bias.data)
    ((h @ b.weight.data + b.bias.data + h @ c.weight.data + c.bias.data) * w).sum().backward()
    assert torch.allclose(gx, xr.grad, atol=1e-5)
    assert torch.allclose(G.node_output("b"), (h @ b.weight.data + b.bias.data).detach(), atol=1e-6)


def test_compute_graph_exporters():
    nn.manual_seed(0)
    G = nn.ComputeGraph([nn.InputSlot("x"), nn.Node("lin", nn.Linear(5, 7), ["x"]), nn.Node("act", nn.Elementwise("tanh"), ["lin"]),
                         nn.Node("b", nn.Linear(7, 3), ["act"]), nn.Node("c", nn.Linear(7, 3), ["act"]),
                         nn.ExternalNode("sum", lambda u, v: u + v, lambda g, u, v: (g, g), ["b", "c"])])
    text = G.describe(nn.TextExporter(), "toy")
    assert "toy: ComputeGraph[1 inputs, 5 nodes]" in text and "lin = Linear[5,7](x)  [42 params]  -> act" in text
    assert "sum = external:<lambda>(b, c)  -> (output)" in text
    mm = G.describe(nn.MermaidExporter())
    assert mm.startswith("flowchart TD") and "n_x --> n_lin" in mm and mm.count("-->") == 6
    rep = nn.FusionReport()
    out = G.describe(rep, "toy")
    assert rep.pairs == [("lin", "act")] and rep.fanout == [("act", 2)] and "fuse lin" in out


def test_schedulers():
    s = nn.schedulers.WarmupCosine(1.0, 10, 110, 0.1)
    assert abs(s(0) - 0.1) < 1e-9 and abs(s(9) - 1.0) < 1e-9
    assert abs(s(60) - (0.1 + 0.45 * (1 + math.cos(math.pi * 0.5)))) < 1e-9
    assert abs(s(500) - 0.1) < 1e-9
    assert nn.schedulers.StepDecay(1.0, 10, 0.5)(25) == 0.25
    assert nn.schedulers.LinearWarmup(2.0, 4)(1) == 1.0
    assert abs(nn.schedulers.Cosine(1.0, 100)(100)) < 1e-12


def test_gpt_backward_fd_tied_and_untied():
    from noeira_b200.models.gpt import GPT
    for tie in (False, True):
        m = GPT(vocab=32, seq=8, dim=16, layers=2, heads=2, tie=tie, seed=1)
        ids = torch.randint(0, 32, (2, 8))
        tgt = torch.randint(0, 32, (2, 8))

        def loss():
            acc = torch.zeros(1)
            nn.cross_entropy(m.forward(ids), tgt, acc)
            return float(acc)
        m.zero_grad()
        acc = torch.zeros(1)
        m.vjp(nn.cross_entropy(m.forward(ids), tgt, acc))
        names = [n for n, _ in m.named_params()]
        assert ("head.weight" in names) != tie and "blocks.1.attn.qkv.weight" in names
        _fd_check(loss, [(n, p) for n, p in m.named_params() if n in ("wte.weight", "wpe.weight", "blocks.0.attn.out.weight",
                                                                      "blocks.1.ffn.0.weight", "ln_f.gamma")], n=4)


def test_vit_backward_fd():
    from noeira_b200.models.gpt import ViT
    m = ViT(image=8, patch=4, dim=16, layers=1, heads=2, classes=5)
    img = torch.randn(3, 3, 8, 8)
    y = torch.tensor([0, 3, 4])

    def loss():
        acc = torch.zeros(1)
        nn.cross_entropy(m.forward(img), y, acc)
        return float(acc)
    m.zero_grad()
    acc = torch.zeros(1)
    m.vjp(nn.cross_entropy(m.forward(img), y, acc))
    _fd_check(loss, [(n, p) for n, p in m.named_params() if n in ("cls_token", "pos_embed", "patch_embed.proj.weight", "head.bias")], n=4)


def test_trainers_reduce_loss_on_cpu():
    from noeira_b200.models.gpt import GPT
    from noeira_b200.training import AutoregressiveTrainer, Trainer
    torch.manual_seed(0)
    x = torch.randn(512, 10)
    y = (x[:, 0] + x[:, 1] > 0).long()
    nn.manual_seed(0)
    model = nn.Sequential(nn.LinearReLU(10, 32), nn.Linear(32, 2, out_fp32=True))
    tr = Trainer(model, x, y, batch=64, lr=1e-2)
    l0, _ = tr.train_epoch(0)
    for e in range(1, 6):
        l1, acc = tr.train_epoch(e)
    assert l1 < 0.6 * l0 and acc > 0.85
    toks = (torch.arange(4000) % 7).long()          # a periodic stream is learnable in a few steps
    lm = GPT(vocab=8, seq=16, dim=32, layers=1, heads=2, seed=0)
    at = AutoregressiveTrainer(lm, toks, batch=8, seq=16, lr=3e-3, warmup=5, total_steps=60)
    at.train_step()
    first = at.mean_loss()
    for _ in range(59):
        at.train_step()
    assert at.mean_loss() / 59 < 0.5 * first
