"""CPU gates for the nn core: explicit VJPs vs torch autograd, arena + optimizers vs torch.optim, naming rules,
checkpoint v3 and safetensors round trips (incl. interop with the `safetensors` library when present)."""
import math
import os
import struct

import pytest
import torch


def test_sequential_vjp_matches_autograd_and_names():
    from noeira_b200 import nn
    nn.manual_seed(0)
    net = nn.Sequential(nn.LinearTanh(17, 64), nn.LinearReLU(64, 64), nn.LinearGELU(64, 32), nn.Linear(32, 3))
    assert [n for n, _ in net.named_params("actor.")][:3] == ["actor.0.weight", "actor.0.bias", "actor.1.weight"]
    x = torch.randn(9, 17)
    y = net(x)
    dx = net.vjp(torch.ones_like(y))
    ws = [p.data.clone().requires_grad_(True) for p in net.params()]
    xx = x.clone().requires_grad_(True)
    h = torch.tanh(xx @ ws[0] + ws[1])
    h = torch.relu(h @ ws[2] + ws[3])
    h = torch.nn.functional.gelu(h @ ws[4] + ws[5], approximate="tanh")
    (h @ ws[6] + ws[7]).sum().backward()
    for p, w in zip(net.params(), ws):
        assert torch.allclose(p.grad, w.grad, atol=1e-5), p.name
    assert torch.allclose(dx, xx.grad, atol=1e-5)
    assert net.params()[0].shape == (17, 64)   # [IN, OUT], the transpose of torch's layout


def test_combinators():
    from noeira_b200 import nn
    nn.manual_seed(1)
    res = nn.Residual(nn.Sequential(nn.LinearTanh(8, 8), nn.Linear(8, 8)))
    assert [n for n, _ in res.named_params()] == ["0.0.weight", "0.0.bias", "0.1.weight", "0.1.bias"]
    x = torch.randn(4, 8)
    y = res(x)
    g = res.vjp(torch.ones_like(y))
    xx = x.clone().requires_grad_(True)
    ws = [p.data for p in res.params()]
    (xx + (torch.tanh(xx @ ws[0] + ws[1]) @ ws[2] + ws[3])).sum().backward()
    assert torch.allclose(g, xx.grad, atol=1e-5)
    par = nn.Parallel(nn.Linear(8, 3), nn.Linear(8, 2))
    out = par(x)
    assert out.shape == (4, 5) and [n for n, _ in par.named_params()][2] == "1.weight"
    assert par.vjp(torch.ones(4, 5)).shape == (4, 8)
    tok = nn.Tokenwise(nn.Linear(8, 6))
    assert tok(torch.randn(2, 5, 8)).shape == (2, 5, 6)
    assert [n for n, _ in tok.named_params()] == ["0.weight", "0.bias"]
    rep = nn.Repeat(3, lambda i: nn.Residual(nn.Linear(8, 8)))
    assert [n for n, _ in rep.named_params()][2] == "1.0.weight"
    ck = nn.Checkpointed(nn.Sequential(nn.LinearTanh(8, 8), nn.Linear(8, 8)))
    ck2 = nn.Sequential(nn.LinearTanh(8, 8), nn.Linear(8, 8))
    ck2.copy_from(ck.inner)
    ck(x)
    ck2(x)
    assert torch.allclose(ck.vjp(torch.ones(4, 8)), ck2.vjp(torch.ones(4, 8)))


def test_arena_adamw_sgd_match_torch():
    from noeira_b200 import nn
    nn.manual_seed(2)
    net = nn.Sequential(nn.Linear(5, 7), nn.Linear(7, 2))
    ref = [torch.nn.Parameter(p.data.clone()) for p in net.params()]
    topt = torch.optim.AdamW([{"params": [ref[0], ref[2]], "weight_decay": 0.1}, {"params": [ref[1], ref[3]], "weight_decay": 0.0}],
                             lr=1e-2, betas=(0.9, 0.999), eps=1e-8)
    opt = nn.AdamW(net.named_params(), lr=1e-2, weight_decay=0.1)
    assert opt.arena.val.data_ptr() == net.params()[0].storage.data_ptr()
    assert opt.arena.numel % 32 == 0
    for step in range(5):
        for p, r in zip(net.params(), ref):
            g = torch.randn(p.shape)
            p.grad.copy_(g)
            r.grad = g.clone()
        opt.step(zero_grad=True)
        topt.step()
    for p, r in zip(net.params(), ref):
        assert torch.allclose(p.data, r.data, atol=1e-6), p.name
    assert float(opt.arena.grd.abs().max()) == 0.0
    # clip: non-finite norm zeroes the step
    net.params()[0].grad.fill_(float("nan"))
    before = opt.arena.val.clone()
    opt.clip(max_norm=1.0)
    assert float(opt.hyper[8]) == 0.0
    opt.arena.grd.nan_to_num_(0.0)
    opt.step()
    assert torch.allclose(before, opt.arena.val, atol=1e-2)


def test_checkpoint_v3_roundtrip_and_validation(tmp_path):
    from noeira_b200 import nn
    from noeira_b200.io import CheckpointError, load_checkpoint, save_checkpoint
    nn.manual_seed(3)
    a = nn.Sequential(nn.LinearTanh(6, 5), nn.Linear(5, 2))
    b = nn.Sequential(nn.LinearTanh(6, 5), nn.Linear(5, 2))
    oa = nn.Adam(a.named_params(), lr=1e-3)
    nn.Adam(b.named_params(), lr=1e-3)
    a.params()[0].grad.fill_(0.5)
    oa.step()
    path = str(tmp_path / "m.ckpt")
    save_checkpoint(path, list(a.named_params()), [], {"step": 2 ** 30 + 1, "lr": 3e-4}, with_moments=True)
    raw = open(path, "rb").read()
    assert raw.startswith(b"storage-ckpt v3\nP 0.weight 30 1\n")
    assert struct.unpack("<f", raw[len(b"storage-ckpt v3\nP 0.weight 30 1\n"):][:4])[0] == pytest.approx(float(a.params()[0].data[0, 0]))
    sc = load_checkpoint(path, list(b.named_params()), [])
    assert sc["step"] == 2 ** 30 + 1 and sc["lr"] == pytest.approx(3e-4)
    for pa, pb in zip(a.params(), b.params()):
        assert torch.equal(pa.data, pb.data) and torch.equal(pa.m, pb.m)
    wrong = nn.Sequential(nn.LinearTanh(6, 4), nn.Linear(4, 2))
    with pytest.raises(CheckpointError):
        load_checkpoint(path, list(wrong.named_params()), [])
    open(path, "wb").write(raw[: len(raw) // 2])
    with pytest.raises(CheckpointError):
        load_checkpoint(path, list(b.named_params()), [])
    assert not os.path.exists(path + ".tmp")


def test_safetensors_roundtrip_validation_and_interop(tmp_path):
    from noeira_b200 import nn
    from noeira_b200.io import SafeTensors, SafeTensorsError, load_safetensors, save_safetensors
    nn.manual_seed(4)
    a, b = nn.Sequential(nn.Linear(4, 3)), nn.Sequential(nn.Linear(4, 3))
    path = str(tmp_path / "m.safetensors")
    assert save_safetensors(path, list(a.named_params())) == 2
    st = SafeTensors(path)
    assert st.metadata["producer"] == "noeira_b200" and st.shape("0.weight") == (12,)
    load_safetensors(path, list(b.named_params()))
    assert torch.equal(a.params()[0].data, b.params()[0].data)
    try:
        from safetensors.numpy import load_file, save_file
        ext = load_file(path)
        assert ext["0.weight"].shape == (12,)
        import numpy as np
        p2 = str(tmp_path / "ext.safetensors")
        save_file({"0.weight": np.arange(12, dtype=np.float32), "0.bias": np.ones(3, dtype=np.float16)}, p2)
        load_safetensors(p2, list(b.named_params()))
        assert float(b.params()[0].data[2, 1]) == 7.0 and float(b.params()[1].data[0]) == 1.0
    except ImportError:
        pass
    raw = bytearray(open(path, "rb").read())
    bad = str(tmp_path / "bad.safetensors")
    open(bad, "wb").write(raw[:-4])
    with pytest.raises(SafeTensorsError):
        SafeTensors(bad)
    raw2 = bytearray(raw)
    raw2[0:8] = struct.pack("<Q", 10 ** 9)
    open(bad, "wb").write(raw2)
    with pytest.raises(SafeTensorsError):
        SafeTensors(bad)
    with pytest.raises(SafeTensorsError):
        load_safetensors(path, [("missing.weight", a.params()[0])], strict=True)


def test_physics_oracle_invariants():
    """Mass matrix symmetric positive definite; free fall accelerates with g; energy conserved without contacts."""
    import numpy as np
    from noeira_b200.physics import oracle, pendulum_cart, planar_chain
    m = planar_chain()
    q = np.random.RandomState(0).uniform(-0.5, 0.5, m.nv)
    M = oracle.mass_matrix(m, q)
    assert np.allclose(M, M.T, atol=1e-10) and np.all(np.linalg.eigvalsh(M) > 0)
    b = oracle.bias_force(m, q, np.zeros(m.nv))
    assert abs(b[1] - m.body_mass.sum() * 9.81) < 1e-4 and abs(b[0]) < 1e-6     # gravity on the root z slide
    pc = pendulum_cart()
    pc.dof_damping[:] = 0
    q, v = np.array([0.0, 2.0]), np.zeros(2)
    warm = np.zeros(pc.nlimit + 3 * pc.ncs)
    def energy(q, v):
        return 0.5 * v @ oracle.mass_matrix(pc, q) @ v + oracle.potential(pc, q)
    e0 = energy(q, v)
    old = pc.opt.timestep
    pc.opt.timestep = 1e-3
    for _ in range(300):
        q, v = oracle.substep(pc, q, v, np.zeros(2), warm)
    pc.opt.timestep = old
    assert abs(energy(q, v) - e0) < 2e-2 * max(1.0, abs(e0))


def test_multi_module_checkpoint_interleaves_params_and_states(tmp_path):
    """Two modules that both carry states: the file holds P… S… of module 0, then P… S… of module 1, then K."""
    from noeira_b200 import nn
    from noeira_b200.io.checkpoint import load_params_multi, save_params_multi
    nn.manual_seed(0)
    mk = lambda: nn.Sequential(nn.Conv2D(3, 4, 3, pad=1), nn.BatchNorm2D(4))
    m0, m1 = mk(), mk()
    for _, s in list(m0.named_states()) + list(m1.named_states()):
        s.data.uniform_(0.5, 1.5)
    path = str(tmp_path / "two.ckpt")
    save_params_multi(path, [m0, m1], {"k": 3.0}, with_moments=False)
    kinds = []
    raw = open(path, "rb").read()
    pos = raw.index(b"\n") + 1
    while pos < len(raw):
        end = raw.index(b"\n", pos)
        parts = raw[pos:end].decode().split(" ")
        kinds.append(parts[0])
        pos = end + 1 + (8 if parts[0] == "K" else 4 * int(parts[2]))
    n_p, n_s = len(list(m0.named_params())), len(list(m0.named_states()))
    assert n_s > 0
    assert kinds == ["P"] * n_p + ["S"] * n_s + ["P"] * n_p + ["S"] * n_s + ["K"]
    a, b = mk(), mk()
    assert load_params_multi(path, [a, b]) == {"k": 3.0}
    for (_, s0), (_, s1) in zip(list(m1.named_states()), list(b.named_states())):
        assert torch.equal(s0.data, s1.data)
