"""PyTorch-named safetensors ↔ this framework's parameters through TorchNameMap (round trip against torch.nn)."""
import numpy as np
import pytest
import torch


def test_torch_named_roundtrip_against_torch_module(tmp_path):
    from noeira_b200 import nn
    from noeira_b200.io.safetensors import SafeTensors, SafeTensorsWriter
    from noeira_b200.nn.torch_names import TN_ZEROS, TorchNameError, TorchNameMap, load_torch_named, mlp_name_map, save_torch_named
    tm = torch.nn.Sequential(torch.nn.Linear(5, 16), torch.nn.Tanh(), torch.nn.Linear(16, 3))
    w = SafeTensorsWriter()
    for k, v in tm.state_dict().items():
        w.add_f32("policy." + k, v.detach().numpy(), list(v.shape))
    w.add_f32("policy.extra.scale", np.ones(2, np.float32), [2])
    path = str(tmp_path / "torch.safetensors")
    w.write(path)
    ours = nn.Sequential(nn.LinearTanh(5, 16), nn.Linear(16, 3))
    m = mlp_name_map([5, 16, 3])
    rep = load_torch_named(path, m, ours.named_params("actor."), prefix="actor.", their_prefix="policy.")
    rep.check()
    assert sorted(rep.loaded) == ["0.bias", "0.weight", "1.bias", "1.weight"] and rep.unclaimed == ["policy.extra.scale"]
    with pytest.raises(TorchNameError):
        rep.check(allow_unclaimed=False)
    x = torch.randn(7, 5)
    assert torch.allclose(ours.forward(x), tm(x), atol=1e-5)                       # [in,out] vs [out,in] handled by the map
    # save back with their names / layouts
    out = str(tmp_path / "back.safetensors")
    assert save_torch_named(out, m, ours.named_params("actor."), prefix="actor.", their_prefix="policy.") == 4
    back = SafeTensors(out)
    for k, v in tm.state_dict().items():
        assert tuple(back.shape("policy." + k)) == tuple(v.shape) and np.allclose(back.get("policy." + k), v.numpy())
    # the failure modes are told apart
    bad = TorchNameMap().add_linear("0.weight", "0.weight", 5, 16)                 # wrong declared shape
    with pytest.raises(TorchNameError, match="shape"):
        load_torch_named(path, bad, ours.named_params("actor."), prefix="actor.", their_prefix="policy.")
    part = TorchNameMap().add_linear("0.weight", "0.weight", 16, 5)
    rep = load_torch_named(path, part, ours.named_params("actor."), prefix="actor.", their_prefix="policy.")
    assert "0.bias" in rep.unmapped
    with pytest.raises(TorchNameError, match="not in the name map"):
        rep.check()
    miss = mlp_name_map([5, 16, 3]).add("2.gamma", "norm.weight", (3,))
    rep = load_torch_named(path, mlp_name_map([5, 16, 3], theirs_fmt="layers.{j}."), ours.named_params("actor."), prefix="actor.",
                           their_prefix="policy.")
    assert len(rep.missing) == 4
    with pytest.raises(TorchNameError):
        TorchNameMap().add("a", "x", (2,)).add("a", "y", (2,))
    z = mlp_name_map([5, 16, 3])
    z.kind[z.index_of_ours("1.bias")] = TN_ZEROS
    ours.mods[1].bias.set_(torch.ones(3))
    rep = load_torch_named(path, z, ours.named_params("actor."), prefix="actor.", their_prefix="policy.")
    assert rep.zeroed == ["1.bias"] and float(ours.mods[1].bias.data.abs().sum()) == 0.0
