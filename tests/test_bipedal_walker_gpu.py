"""BipedalWalker CUDA kernel against the host build of the same source, long-run sanity, PPO on the device rollout."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_kernel_matches_host_oracle():
    from noeira_b200.envs import BipedalWalkerEnv
    n = 256
    g, c = BipedalWalkerEnv(n, device="cuda", seed=11), BipedalWalkerEnv(n, device="cpu", seed=11)
    og, oc = g.reset_batch(), c.reset_batch()
    assert torch.allclose(og.cpu(), oc, atol=1e-5)
    gen = torch.Generator().manual_seed(0)
    for step in range(10):
        a = torch.rand(n, 4, generator=gen) * 2 - 1
        g.step_batch(a.cuda(), auto_reset=False)
        c.step_batch(a, auto_reset=False)
        # dozens of dependent solver sweeps per step: FMA contraction differs between nvcc and g++, and a foot that touches
        # down one step earlier in one build flips a contact flag and sends that lane elsewhere.  The first steps agree
        # everywhere; later nearly all lanes still agree closely
        per_env = (g.next_obs.cpu() - c.next_obs).abs().max(1).values
        if step < 4:
            assert float(per_env.max()) < 5e-3, (step, float(per_env.max()))
        assert float((per_env < 2e-2).float().mean()) > 0.95, (step, float((per_env < 2e-2).float().mean()))
        assert float((g.done.cpu() == c.done).float().mean()) > 0.98


def test_long_run_statistics_and_ppo_rollout():
    from noeira_b200.agents.ppo import PPOConfig, PPOTrainer
    from noeira_b200.envs import BipedalWalkerEnv
    env = BipedalWalkerEnv(2048, device="cuda", seed=2)
    env.reset_batch()
    for _ in range(300):
        env.step_batch(torch.rand(2048, 4, device="cuda") * 2 - 1)
    torch.cuda.synchronize()
    assert torch.isfinite(env.obs).all() and torch.isfinite(env.reward).all()
    assert torch.allclose(env.obs_bf16[:, :24].float(), env.obs, atol=3e-2, rtol=1e-2)
    episodes = float(env.ep_stats[1])
    assert episodes > 1000 and -140 < float(env.ep_stats[0]) / episodes < -80          # a random policy falls over
    env2 = BipedalWalkerEnv(1024, device="cuda", seed=0)
    agent = PPOTrainer(env2, PPOConfig(n_envs=1024, rollout_len=32, n_epochs=4, n_minibatches=8))
    for _ in range(4):
        m = agent.train_iteration()
    assert all(map(lambda v: v == v, (m["policy_loss"], m["value_loss"], m["entropy"]))) and m["episodes"] > 0
