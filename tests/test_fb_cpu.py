"""Forward-backward representations: reward-free training on Pendulum transitions and zero-shot task inference."""
import torch


def test_fb_trains_reward_free_and_infers_task_vectors():
    from noeira_b200.agents.fb import FBAgent, FBConfig
    from noeira_b200.envs import PendulumEnv
    env = PendulumEnv(16, seed=0)
    obs = env.reset_batch().float().clone()
    S, A, SP = [], [], []
    g = torch.Generator().manual_seed(0)
    for _ in range(150):
        a = torch.rand(16, 1, generator=g) * 2 - 1
        nxt, r, done, term = env.step_batch(a)
        S.append(obs), A.append(a), SP.append(env.next_obs.float().clone())
        obs = nxt.float().clone()
    S, A, SP = torch.cat(S), torch.cat(A), torch.cat(SP)
    ag = FBAgent(FBConfig(obs_dim=3, act_dim=1, z_dim=8, hidden=64, batch=96, lr=1e-3, seed=0))
    hist = []
    for it in range(120):
        idx = torch.randint(0, S.shape[0], (96,), generator=g)
        hist.append(ag.update(S[idx], A[idx], SP[idx]))
    assert all(v == v for v in hist[-1].values())
    # the backward map spreads out: normalised rows whose Gram matrix moved towards the identity scale
    B = ag.backward_map(ag.b, S[:256], ag._fwd)
    assert torch.allclose(B.norm(dim=-1), torch.full((256,), 8 ** 0.5), atol=1e-4)
    assert hist[-1]["fb_loss"] < hist[0]["fb_loss"]
    # zero-shot: two opposite rewards give (nearly) opposite task vectors; the predicted value of the inferred task
    # correlates with the reward it was inferred from
    r_up = S[:, 0]                                  # cos θ: upright is good
    z_up, z_down = ag.infer_z(S, r_up), ag.infer_z(S, -r_up)
    assert abs(float(z_up.norm()) - 8 ** 0.5) < 1e-4 and float(torch.dot(z_up, z_down)) < -7.9
    proj = (ag.backward_map(ag.b, S, ag._fwd) * z_up).sum(-1)
    corr = torch.corrcoef(torch.stack([proj, r_up]))[0, 1]
    assert float(corr) > 0.3, float(corr)
    a = ag.select_action(S[:5], z_up)
    assert a.shape == (5, 1) and float(a.abs().max()) <= 1.0
    assert ag.fb_opt.arena.grd.abs().max().item() == 0.0
