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
        u = env.render(res, uint8=True)
        assert u.dtype == torch.uint8 and torch.equal(u, (a * 255.0 + 0.5).to(torch.uint8)) and set(u.unique().tolist()) <= {77, 179, 255}


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


def test_fused_environment_step_matches_the_tensor_program_including_resets():
    """One launch per step: dynamics, reward, time limit, statistics, both observations and the reset, against the same step
    assembled from the tensor program (the reset's track choice is read back from the kernel's new state)."""
    from noeira_b200.envs.car_racing import HDR, CarRacingEnv, scripted_driver
    from noeira_b200.ops import check_status
    N = 96
    k = CarRacingEnv(N, device="cuda", seed=4, lookahead=5, n_tracks=6)
    e = CarRacingEnv(N, device="cuda", seed=4, lookahead=5, n_tracks=6)
    e.use_kernels = False
    k.max_steps = 37                                                   # time-limit resets within the test
    k.reset_batch()
    g = torch.Generator(device="cuda").manual_seed(1)
    n_done, r_sum = 0, 0.0
    for step in range(100):
        a = scripted_driver(k, target_speed=45.0) + 0.3 * torch.randn(N, 3, device="cuda", generator=g)
        s, steps, ret = k.state.clone(), k.steps.clone(), k.ep_return.clone()
        obs, r, d, tm = k.step_batch(a)
        s2, r_ref, t_ref = e._dynamics_tensor(s, a)
        done_ref = t_ref | (steps + 1 >= 37)
        assert torch.equal(d > 0.5, done_ref) and torch.equal(tm > 0.5, t_ref) and (r - r_ref).abs().max() < 1e-4, step
        tol = 2e-3 * max(1.0, float(s2[:, :16].abs().max()))
        assert (k.pre_reset_state[:, :16] - s2[:, :16]).abs().max() < tol and torch.equal(k.pre_reset_state[:, 16:], s2[:, 16:])
        assert (k.next_obs - e._observe(k.pre_reset_state)).abs().max() < 1e-3
        assert (k.obs - e._observe(k.state)).abs().max() < 1e-3
        keep = ~done_ref
        assert torch.equal(k.state[keep], k.pre_reset_state[keep])
        if done_ref.any():
            new = k.state[done_ref]
            tid = new[:, 12].long()
            assert (tid >= 0).all() and (tid < 6).all() and torch.equal(new[:, 0:2], k.track[tid, 0])
            assert float(new[:, 3:12].abs().max()) == 0 and float(new[:, 13:].abs().sum()) == 0
            assert float(k.steps[done_ref].abs().max()) == 0 and float(k.ep_return[done_ref].abs().max()) == 0
            assert (k.finished_return[done_ref] - (ret + r)[done_ref]).abs().max() < 1e-3
        assert torch.equal(k.steps[keep], steps[keep] + 1)
        n_done += int(done_ref.sum())
        r_sum += float(r.sum())
    torch.cuda.synchronize()
    check_status()
    st = k.ep_stats.tolist()
    assert n_done >= 2 * N and st[1] == n_done and st[3] == 100 * N and abs(st[2] - r_sum) < 1e-3 * max(1.0, abs(r_sum))
    assert len(torch.unique(k.state[:, 12])) > 1                        # resets draw different tracks
    # bf16 rows for the on-policy trainer
    ob, nb = torch.zeros(N, 64, device="cuda", dtype=torch.bfloat16), torch.zeros(N, 64, device="cuda", dtype=torch.bfloat16)
    k.step(a, k.reward, k.done, k.terminated, obs_bf16=ob, next_obs_bf16=nb, ep_stats=k.ep_stats)
    assert (ob[:, :23].float() - e._observe(k.state)).abs().max() < 0.02 * max(1.0, float(e._observe(k.state).abs().max()))
    assert float(ob[:, 23:].abs().max()) == 0


def test_ppo_learns_to_drive_from_captured_rollouts():
    """The in-place fused step lets rollout and update replay from CUDA graphs; 130 iterations of 32 x 4096 steps take the
    reward per step from the idle level (about −0.1 + the first tiles) to several tiles per ten steps."""
    from noeira_b200.agents.ppo import PPOConfig, PPOTrainer
    from noeira_b200.envs.car_racing import CarRacingEnv
    env = CarRacingEnv(4096, device="cuda", seed=0, lookahead=8)
    tr = PPOTrainer(env, PPOConfig(n_envs=4096, rollout_len=32, n_epochs=4, n_minibatches=8, hidden=256, entropy_coef=1e-3, seed=0))
    hist = [float(tr.train_iteration()["mean_step_reward"]) for _ in range(130)]
    early, late = sum(hist[10:30]) / 20, sum(hist[-10:]) / 10
    assert tr._graphs and late > 0.4 and late > early + 0.3, (early, late)
    assert float(env.visited_fraction().max()) > 0.3


def test_ppo_steps_a_classic_tensor_environment_without_graphs():
    from noeira_b200.agents.ppo import PPOConfig, PPOTrainer
    from noeira_b200.envs import PendulumEnv
    env = PendulumEnv(512, device="cuda", seed=0)
    tr = PPOTrainer(env, PPOConfig(n_envs=512, rollout_len=16, n_epochs=2, n_minibatches=4, seed=0))
    assert tr.cfg.use_cuda_graphs is False                          # the environment declares itself unsafe to capture
    m = [tr.train_iteration() for _ in range(3)][-1]
    assert torch.isfinite(torch.as_tensor(float(m["policy_loss"]))) and -17.0 < float(m["mean_step_reward"]) < 0.0
