"""SAC / TD3 updates on CUDA (bf16 tensor-core path): finite, and the critic fits a fixed batch."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _batch(dev):
    g = torch.Generator().manual_seed(0)
    B = 256
    s, sp = torch.randn(B, 17, generator=g), torch.randn(B, 17, generator=g)
    a = torch.rand(B, 6, generator=g) * 2 - 1
    r = torch.randn(B, generator=g)
    d = (torch.rand(B, generator=g) < 0.01).float()
    return tuple(t.to(dev) for t in (s, a, r, sp, d))


def test_sac_update_cuda_matches_cpu_first_step_and_learns():
    from noeira_b200.agents.sac import SACConfig, SACTrainer
    cpu, gpu = SACTrainer(SACConfig(seed=3), device="cpu"), SACTrainer(SACConfig(seed=3), device="cuda")
    mc = cpu.update(*_batch("cpu"))
    mg = gpu.update(*_batch("cuda"))
    assert abs(float(mc["critic_loss"]) - float(mg["critic_loss"])) < 0.05 * max(1.0, abs(float(mc["critic_loss"])))
    first = float(mg["critic_loss"])
    for _ in range(150):
        mg = gpu.update(*_batch("cuda"))
    assert all(torch.isfinite(torch.as_tensor(float(v))) for v in mg.values())
    assert float(mg["critic_loss"]) < 0.7 * first


def test_td3_update_cuda():
    from noeira_b200.agents.sac import TD3Config, TD3Trainer
    tr = TD3Trainer(TD3Config(seed=1), device="cuda")
    first = None
    for i in range(100):
        m = tr.update(*_batch("cuda"))
        first = first if first is not None else float(m["critic_loss"])
    assert float(m["critic_loss"]) < 0.8 * first
    a = tr.select_action(_batch("cuda")[0])
    assert a.shape == (256, 6) and a.abs().max() <= 1.0 + 1e-6


def test_sac_captured_update_tracks_eager():
    from noeira_b200.agents.sac import SACConfig, SACTrainer
    a, b = SACTrainer(SACConfig(seed=4), device="cuda"), SACTrainer(SACConfig(seed=4), device="cuda")
    batch = _batch("cuda")
    la, lb = [], []
    for _ in range(12):
        la.append(float(a.update(*batch)["critic_loss"]))
        lb.append(float(b.update_captured(*batch)["critic_loss"]))
    assert b._graphed.graph is not None and b._graphed.launches > 50 and b.total_train_steps == 12
    assert all(abs(x - y) <= 2e-2 * max(1.0, abs(x)) for x, y in zip(la, lb)), (la, lb)
    assert lb[-1] < lb[0]


def test_sac_kernel_path_matches_the_eager_tensor_path():
    """The glue kernels (sampling, target, critic gradients, critic choice, squashed-Gaussian backward) against the same
    update written with tensor operations: same noise stream, same parameters after every step to bf16 tolerance."""
    from noeira_b200.agents.sac import SACConfig, SACTrainer
    from noeira_b200.ops import check_status
    k, e = SACTrainer(SACConfig(seed=5), device="cuda"), SACTrainer(SACConfig(seed=5), device="cuda")
    e.use_kernels = False
    batch = _batch("cuda")
    for step in range(5):
        mk, me = k.update(*batch), e.update(*batch)
        torch.cuda.synchronize()
        check_status()
        for key in ("critic_loss", "actor_loss", "mean_q", "mean_logp"):
            assert abs(float(mk[key]) - float(me[key])) < 2e-2 * max(1.0, abs(float(me[key]))), (step, key, float(mk[key]), float(me[key]))
    for a, b in ((k.actor_opt, e.actor_opt), (k.critic_opt, e.critic_opt)):
        assert (a.arena.val - b.arena.val).abs().max().item() < 3e-3
    assert abs(float(k.alpha) - float(e.alpha)) < 1e-5
    # bit-repeatable: two kernel-path trainers from the same seed stay identical
    k2 = SACTrainer(SACConfig(seed=5), device="cuda")
    for _ in range(5):
        k2.update(*batch)
    assert torch.equal(k2.actor_opt.arena.val, k.actor_opt.arena.val) and torch.equal(k2.critic_opt.arena.val, k.critic_opt.arena.val)


def test_td3_kernel_path_matches_the_eager_tensor_path():
    from noeira_b200.agents.sac import TD3Config, TD3Trainer
    from noeira_b200.ops import check_status
    k, e = TD3Trainer(TD3Config(seed=2), device="cuda"), TD3Trainer(TD3Config(seed=2), device="cuda")
    e.use_kernels = False
    batch = _batch("cuda")
    for step in range(6):
        mk, me = k.update(*batch), e.update(*batch)
        torch.cuda.synchronize()
        check_status()
        assert set(mk) == set(me)
        for key in mk:
            assert abs(float(mk[key]) - float(me[key])) < 2e-2 * max(1.0, abs(float(me[key]))), (step, key, float(mk[key]), float(me[key]))
    for a, b in ((k.actor_opt, e.actor_opt), (k.critic_opt, e.critic_opt)):
        assert (a.arena.val - b.arena.val).abs().max().item() < 3e-3
