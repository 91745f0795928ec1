"""Fused physics step kernel against the float64 NumPy oracle (different derivation of M and bias)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(model_fn, env_cls_task, steps, action_scale, tol_q, tol_v):
    from noeira_b200.envs import Physics3dBatchedEnv
    from noeira_b200.physics import oracle
    from noeira_b200.physics.engine import TaskSpec
    m = model_fn()
    task = TaskSpec(frame_skip=5, max_steps=100000)
    n = 64
    env = Physics3dBatchedEnv(m, n, task, seed=3)
    env.reset_batch()
    torch.cuda.synchronize()
    rng = np.random.RandomState(0)
    qpos = env.engine.qpos.cpu().double().numpy().copy()
    qvel = env.engine.qvel.cpu().double().numpy().copy()
    check_envs = [0, 1, 17]
    warm = {e: np.zeros(m.nlimit + 3 * m.ncs) for e in check_envs}
    q = {e: qpos[e].copy() for e in check_envs}
    v = {e: qvel[e].copy() for e in check_envs}
    dbg = torch.zeros(m.nv * m.nv + 3 * m.nv + 4, device="cuda")
    for s in range(steps):
        act = (rng.uniform(-1, 1, size=(n, m.nu)) * action_scale).astype(np.float32)
        a_t = torch.from_numpy(act).cuda()
        env.step_batch(a_t, dbg=dbg if s == 0 else None)
        torch.cuda.synchronize()
        for e in check_envs:
            d = {} if (s == 0 and e == 0) else None
            q[e], v[e] = oracle.env_step(m, q[e], v[e], act[e], warm[e], frame_skip=5, debug=d)
            if d is not None:
                nv = m.nv
                g = dbg.cpu().double().numpy()
                M_k = g[: nv * nv].reshape(nv, nv)
                assert np.allclose(M_k, d["M"], atol=2e-4 * max(1, np.abs(d["M"]).max())), (M_k, d["M"])
                assert np.allclose(g[nv * nv: nv * nv + nv], d["bias"], atol=2e-3 * max(1, np.abs(d["bias"]).max()))
                assert np.allclose(g[nv * nv + nv: nv * nv + 2 * nv], d["qacc_smooth"],
                                   atol=2e-3 * max(1, np.abs(d["qacc_smooth"]).max()))
                assert int(g[nv * nv + 3 * nv]) == d["nrow"]
                assert np.allclose(g[nv * nv + 2 * nv: nv * nv + 3 * nv], d["qacc"], atol=5e-3 * max(1, np.abs(d["qacc"]).max()))
        kq = env.engine.qpos.cpu().double().numpy()
        kv = env.engine.qvel.cpu().double().numpy()
        for e in check_envs:
            assert np.allclose(kq[e], q[e], atol=tol_q), (s, e, kq[e], q[e])
            assert np.allclose(kv[e], v[e], atol=tol_v), (s, e, kv[e], v[e])
    assert torch.isfinite(env.obs).all() and torch.isfinite(env.reward).all()


def test_planar_chain_matches_oracle():
    from noeira_b200.physics import planar_chain
    _run(planar_chain, None, steps=6, action_scale=0.3, tol_q=5e-3, tol_v=8e-2)


def test_half_cheetah_matches_oracle():
    from noeira_b200.physics import half_cheetah
    _run(half_cheetah, None, steps=6, action_scale=0.5, tol_q=5e-3, tol_v=8e-2)


@pytest.mark.parametrize("name,scale", [("walker2d", 0.3), ("inverted_double_pendulum", 0.05), ("reacher", 0.05), ("hopper", 0.3)])
def test_more_models_match_oracle(name, scale):
    from noeira_b200 import physics
    _run(getattr(physics, name), None, steps=4, action_scale=scale, tol_q=5e-3, tol_v=8e-2)


def test_new_envs_step_and_terminate():
    from noeira_b200.envs import InvertedDoublePendulumEnv, InvertedPendulumEnv, ReacherEnv, Walker2dEnv
    for cls, act in ((Walker2dEnv, 6), (InvertedDoublePendulumEnv, 1), (InvertedPendulumEnv, 1), (ReacherEnv, 2)):
        env = cls(256, seed=0)
        assert env.act_dim == act
        env.reset_batch()
        for _ in range(120):
            env.step_batch(torch.rand(256, act, device="cuda") * 2 - 1)
        torch.cuda.synchronize()
        assert torch.isfinite(env.obs).all() and torch.isfinite(env.reward).all(), cls.__name__
        assert float(env.ep_stats[1]) > 0, cls.__name__                  # random actions end episodes (falls / time limits)


def test_free_fall_and_rest():
    """No actuation: the chain falls with g until contact, then rests on the plane at z = radius."""
    from noeira_b200.envs import PlanarChainEnv
    env = PlanarChainEnv(256, seed=1)
    env.reset_batch()
    a = torch.zeros(256, 6, device="cuda")
    for _ in range(120):
        env.step_batch(a)
    torch.cuda.synchronize()
    xpos, _ = env.engine.body_poses()
    z = xpos[:, :, 2]
    assert torch.isfinite(z).all()
    assert (z > 0.03).all() and (z < 0.06).all(), (z.min().item(), z.max().item())
    assert env.engine.qvel.abs().max().item() < 0.05


def test_env_reset_on_truncation_and_determinism():
    from noeira_b200.envs import PlanarChainEnv
    outs = []
    for _ in range(2):
        env = PlanarChainEnv(128, seed=5, max_steps=7)
        env.reset_batch()
        g = torch.Generator(device="cuda").manual_seed(0)
        dones = 0
        for _ in range(15):
            a = torch.rand(128, 6, device="cuda", generator=g) * 2 - 1
            env.step_batch(a)
            dones += int(env.done.sum().item())
        outs.append((env.obs.clone(), env.engine.qpos.clone()))
        assert dones == 2 * 128
        assert int(env.engine.step_count.max().item()) == 1
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
