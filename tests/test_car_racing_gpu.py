"""Car racing on CUDA: the fused step kernel and the camera kernel against the tensor-program oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_step_kernel_matches_the_tensor_program_along_a_driven_rollout():
    from noeira_b200.envs.car_racing import CarRacingEnv, scripted_driver
    from noeira_b200.ops import check_status
    k = CarRacingEnv(64, device="cuda", seed=1)
    e = CarRacingEnv(64, device="cuda", seed=1)
    e.use_kernels = False
    k.reset_batch(), e.reset_batch()
    assert torch.equal(k.state, e.state)
    g = torch.Generator(device="cuda").manual_seed(0)
    for step in range(150):
        a = scripted_driver(e, target_speed=45.0) + 0.3 * torch.randn(64, 3, device="cuda", generator=g)
        # each step starts from the oracle's state, so that the comparison is per step and not of two chaotic rollouts
        sk, rk, tk = k._dynamics_kernel(e.state, a)
        se, re, te = e._dynamics_tensor(e.state, a)
        assert (sk[:, :16] - se[:, :16]).abs().max() < 2e-3 * max(1.0, float(se[:, :16].abs().max())), step
        assert torch.equal(sk[:, 16:], se[:, 16:]) and torch.equal(tk, te)
        assert (rk - re).abs().max() < 1e-4
        e.step_batch(a, auto_reset=True)
    torch.cuda.synchronize()
    check_status()
    assert float(e.state[:, 13].max()) > 30


def test_camera_kernel_matches_the_tensor_program():
    from noeira_b200.envs.car_racing import CarRacingEnv, scripted_driver
    env = CarRacingEnv(16, device="cuda", seed=2)
    env.reset_batch()
    for _ in range(120):
        env.step_batch(scripted_driver(env), auto_reset=False)
    for res in (96, 64):
        a = env.render(res)
        env.use_kernels = False
        b = env.render(res)
        env.use_kernels = True
        # pixels whose centre lies within rounding of the road edge may differ
        assert (a != b).float().mean() < 2e-3
        assert (a == 0.7).float().mean() > 0.1 and (a == 1.0).any()


def test_full_environment_loop_with_resets_and_pixels():
    from noeira_b200.envs.car_racing import CarRacingPixelEnv
    env = CarRacingPixelEnv(32, device="cuda", seed=3, res=64)
    obs = env.reset_batch()
    total = torch.zeros(32, device="cuda")
    for t in range(60):
        obs, r, d, tm = env.step_batch(torch.full((32,), 3, device="cuda"))
        total += r
    assert obs.shape == (32, 4, 64, 64) and torch.isfinite(total).all() and float(total.max()) > 0


def test_ppo_drives_the_tensor_environment_through_its_engine_surface():
    """PPO steps ``env.engine`` into its rollout buffers; tensor-program environments offer that surface too."""
    from noeira_b200.agents.ppo import PPOConfig, PPOTrainer
    from noeira_b200.envs.car_racing import CarRacingEnv
    env = CarRacingEnv(256, device="cuda", seed=0, lookahead=6)
    cfg = PPOConfig(n_envs=256, rollout_len=16, n_epochs=2, n_minibatches=4, use_cuda_graphs=False, seed=0)
    tr = PPOTrainer(env, cfg)
    for _ in range(3):
        m = tr.train_iteration()
    assert all(torch.isfinite(torch.as_tensor(float(m[k]))) for k in ("policy_loss", "value_loss", "entropy", "mean_step_reward"))
    assert float(env.state[:, 13].max()) >= 1                                # cars moved over at least a tile
