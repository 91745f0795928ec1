import pytest
import torch

pytestmark = pytest.mark.gpu


def _trainer(graphs, n=256):
    from noeira_b200.agents.ppo import PPOConfig, PPOTrainer
    from noeira_b200.envs import PlanarChainEnv
    env = PlanarChainEnv(n, seed=3)
    cfg = PPOConfig(n_envs=n, rollout_len=8, n_epochs=2, n_minibatches=2, hidden=256, seed=1, use_cuda_graphs=graphs)
    return PPOTrainer(env, cfg)


def test_ppo_iteration_runs_and_learns_something():
    from noeira_b200.ops import check_status
    tr = _trainer(True)
    w0 = tr.actor.params()[0].data.clone()
    stats = None
    for _ in range(4):
        stats = tr.train_iteration()
    torch.cuda.synchronize()
    check_status()
    assert all(v == v or k == "mean_episode_return" for k, v in stats.items()), stats
    assert not torch.equal(w0, tr.actor.params()[0].data)
    assert torch.isfinite(tr.actor_opt.arena.val).all() and torch.isfinite(tr.critic_opt.arena.val).all()
    assert abs(stats["entropy"] - 6 * (0.5 * (1.8378770664 + 1) - 0.5)) < 0.2
    assert stats["clip_frac"] < 0.9


def test_ppo_graph_replay_equals_eager():
    """Captured phases must reproduce the eager enqueue sequence bit for bit
    (the reference gates this in tests/nn/test_ppo_train_graph_parity.mojo)."""
    a, b = _trainer(False), _trainer(True)
    for _ in range(3):
        a.train_iteration(read_metrics=False)
        b.train_iteration(read_metrics=False)
    torch.cuda.synchronize()
    assert torch.equal(a.actor_opt.arena.val, b.actor_opt.arena.val)
    assert torch.equal(a.critic_opt.arena.val, b.critic_opt.arena.val)
    assert torch.equal(a.env.engine.qpos, b.env.engine.qpos)


def test_ppo_actor_gradient_matches_autograd():
    """One minibatch: gradients of the clipped surrogate through our kernels vs torch autograd in fp32."""
    import math
    tr = _trainer(False)
    tr.collect()
    tr.actor_opt.zero_grad()
    env, cfg = tr.env, tr.cfg
    import ctypes
    from noeira_b200._native import check, ptr, stream_ptr
    lib = tr.lib
    check(lib.nb_ppo_counter(ptr(tr.counters), ctypes.c_int(0), ctypes.c_int(1), stream_ptr()), "c")
    check(lib.nb_ppo_gather(ptr(tr.obs_buf), ctypes.c_int(env.obs_pad * 2), ptr(tr.act_buf), ctypes.c_int(tr.AP),
                            ptr(tr.logp_buf), ptr(tr.adv_buf), ptr(tr.ret_buf), ptr(tr.mb_obs), ptr(tr.mb_act),
                            ptr(tr.mb_logp), ptr(tr.mb_adv), ptr(tr.mb_ret), ptr(tr.partials), ptr(tr.adv_stats),
                            ctypes.c_int(tr.pool), ctypes.c_int(tr.mb), ctypes.c_int(cfg.n_minibatches),
                            ctypes.c_ulonglong(5), ptr(tr.counters), stream_ptr()), "g")
    torch.cuda.synchronize()
    # the gather is a permutation prefix: every gathered row exists in the pool
    pool_obs = tr.obs_buf[: cfg.rollout_len].reshape(tr.pool, -1)
    assert (tr.mb_obs[:16, None, :17].float() - pool_obs[None, :, :17].float()).abs().sum(-1).min(1).values.max() == 0
    head = tr.actor.mods[2]
    mu = tr.actor.forward(tr.mb_obs)
    check(lib.nb_ppo_objective(ptr(mu), ctypes.c_int(mu.stride(0)), ptr(head.log_std.storage), ptr(tr.mb_act),
                               ctypes.c_int(tr.AP), ptr(tr.mb_logp), ptr(tr.mb_adv), ptr(tr.adv_stats), ptr(tr.dmu),
                               ctypes.c_int(tr.AP), ptr(tr.partials), ptr(tr.partials2), ptr(head.log_std.grad_storage),
                               ptr(tr.metrics), ctypes.c_int(tr.mb), ctypes.c_int(env.act_dim), ctypes.c_float(0.2),
                               ctypes.c_float(0.01), ctypes.c_float(1.0 / tr.mb), stream_ptr()), "o")
    tr.actor.vjp(tr.dmu[:, : env.act_dim])
    torch.cuda.synchronize()
    # fp32 torch reference on the same minibatch
    ps = [p.data.clone().double().requires_grad_(True) for p in tr.actor.params()]
    W0, b0, W1, b1, W2, b2, ls = ps
    x = tr.mb_obs[:, :17].double()
    h = torch.tanh(torch.tanh(x @ W0 + b0) @ W1 + b1)
    m = h @ W2 + b2
    MB = m.shape[0]
    m.register_hook(lambda g: (g * MB).clamp(-10, 10) / MB)   # per-element gradient clip of the objective
    lsb = ls.expand(MB, -1)
    lsb.register_hook(lambda g: (g * MB).clamp(-10, 10) / MB)
    lsc = lsb.clamp(-5, 2)
    sd = lsc.exp() + 1e-6
    act = tr.mb_act[:, : env.act_dim].double()
    lp = (-0.5 * (math.log(2 * math.pi) + 2 * lsc + ((act - m) / sd) ** 2)).sum(1)
    A = (tr.mb_adv.double() - tr.mb_adv.double().mean()) / (tr.mb_adv.double().std(unbiased=False) + 1e-8)
    ratio = (lp - tr.mb_logp.double()).clamp(-20, 20).exp()
    loss = -torch.min(ratio * A, ratio.clamp(0.8, 1.2) * A) - 0.01 * (0.5 * (math.log(2 * math.pi) + 1) + lsc).sum(1)
    loss.mean().backward()
    for p, r in zip(tr.actor.params(), ps):
        g, rg = p.grad.double(), r.grad
        denom = rg.abs().max().item() + 1e-8
        assert (g - rg).abs().max().item() / denom < 0.06, (p.name, (g - rg).abs().max().item(), denom)


def test_steady_state_iteration_allocates_nothing():
    """After warm-up and capture, a PPO iteration is graph replays only: the caching allocator is not entered."""
    import torch
    from noeira_b200.agents.ppo import PPOConfig, PPOTrainer
    from noeira_b200.envs import PlanarChainEnv
    from noeira_b200.utils.trace import AllocTracer
    env = PlanarChainEnv(512, seed=3)
    tr = PPOTrainer(env, PPOConfig(n_envs=512, rollout_len=4, n_epochs=1, n_minibatches=2))
    for _ in range(3):
        tr.train_iteration(read_metrics=False)
    torch.cuda.synchronize()
    tracer = AllocTracer(enabled=True)
    with tracer.scope("iteration"):
        tr.train_iteration(read_metrics=False)
        torch.cuda.synchronize()
    tracer.assert_steady("iteration")


def test_ppo_tf32_precision_arm_tracks_the_bf16_arm():
    """The same iterations with the policy / value networks on the TF32 path (fp32 activations and weights, layer by
    layer) and on the fused bf16 path: both finite, same entropy, first-iteration losses close."""
    from noeira_b200.agents.ppo import PPOConfig, PPOTrainer
    from noeira_b200.envs import PlanarChainEnv
    from noeira_b200.ops import check_status
    out = {}
    for prec in ("bf16", "tf32"):
        env = PlanarChainEnv(1024, seed=3)
        tr = PPOTrainer(env, PPOConfig(n_envs=1024, rollout_len=8, n_epochs=2, n_minibatches=2, hidden=256, seed=1,
                                       precision=prec))
        first = tr.train_iteration()
        for _ in range(2):
            last = tr.train_iteration()
        torch.cuda.synchronize()
        check_status()
        assert torch.isfinite(tr.actor_opt.arena.val).all() and torch.isfinite(tr.critic_opt.arena.val).all()
        out[prec] = (first, last)
    a, b = out["bf16"][0], out["tf32"][0]
    assert abs(a["entropy"] - b["entropy"]) < 1e-3
    assert abs(a["value_loss"] - b["value_loss"]) < 0.1 * max(1.0, abs(a["value_loss"])), (a, b)


def test_ppo_learns_the_planar_chain_task():
    """Convergence gate: the mean reward per step of the planar-chain locomotion task starts negative and must be clearly
    positive after 50 iterations of 1024 envs x 32 steps (measured: about -0.3 at the start, 1.4 to 1.7 at iteration 50,
    above 4 at iteration 80, for two seeds)."""
    from noeira_b200.agents.ppo import PPOConfig, PPOTrainer
    from noeira_b200.envs import PlanarChainEnv
    env = PlanarChainEnv(1024, seed=1)
    tr = PPOTrainer(env, PPOConfig(n_envs=1024, rollout_len=32, n_epochs=4, n_minibatches=8, hidden=256, seed=1))
    first = tr.train_iteration()["mean_step_reward"]
    for _ in range(49):
        last = tr.train_iteration()
    assert first < 0.0 and last["mean_step_reward"] > 0.5, (first, last)
    assert last["mean_step_reward"] > first + 0.8
