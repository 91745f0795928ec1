"""LunarLander CUDA kernel against the host build of the same source, and a short PPO run on it."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_kernel_matches_host_oracle():
    from noeira_b200.envs.lunar_lander import LunarLanderEnv
    n = 256
    g, c = LunarLanderEnv(n, device="cuda", seed=11), LunarLanderEnv(n, device="cpu", seed=11)
    og, oc = g.reset_batch(), c.reset_batch()
    assert torch.allclose(og.cpu(), oc, atol=1e-6)
    gen = torch.Generator().manual_seed(0)
    for step in range(12):
        a = torch.rand(n, 2, generator=gen) * 2 - 1
        g.step_batch(a.cuda(), auto_reset=False)
        c.step_batch(a, auto_reset=False)
        # the solver runs 180 dependent sweeps per step: FMA contraction differs between nvcc and g++, so lanes drift apart
        # slowly; twelve steps stay within 1e-3
        assert torch.allclose(g.next_obs.cpu(), c.next_obs, atol=2e-3), (step, (g.next_obs.cpu() - c.next_obs).abs().max())
        assert torch.allclose(g.reward.cpu(), c.reward, atol=0.2)
        assert torch.equal(g.done.cpu(), c.done)


def test_long_run_statistics_and_bf16_mirror():
    from noeira_b200.envs.lunar_lander import LunarLanderEnv
    env = LunarLanderEnv(2048, device="cuda", seed=2)
    env.reset_batch()
    for _ in range(300):
        env.step_batch(torch.rand(2048, 2, device="cuda") * 2 - 1)
    torch.cuda.synchronize()
    assert torch.isfinite(env.obs).all() and torch.isfinite(env.reward).all()
    assert torch.allclose(env.obs_bf16[:, :8].float(), env.obs, atol=2e-2, rtol=1e-2)
    episodes = float(env.ep_stats[1])
    assert episodes > 2048                                    # random thrust crashes within ~100 steps
    assert -400 < float(env.ep_stats[0]) / episodes < -50     # mean return of a random policy


def test_ppo_device_rollout_runs_on_lunar_lander():
    from noeira_b200.agents.ppo import PPOConfig, PPOTrainer
    from noeira_b200.envs.lunar_lander import LunarLanderEnv
    env = LunarLanderEnv(1024, device="cuda", seed=0)
    agent = PPOTrainer(env, PPOConfig(n_envs=1024, rollout_len=32, n_epochs=4, n_minibatches=8))
    m0 = agent.train_iteration()
    for _ in range(5):
        m = agent.train_iteration()
    assert all(map(lambda v: v == v, (m["policy_loss"], m["value_loss"], m["entropy"])))   # finite
    assert m["episodes"] > 0
