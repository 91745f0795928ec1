"""ACT deployment pieces: temporal ensemble weights, norm.json round trip, closed-loop policy on the CPU oracle path."""
import math

import numpy as np
import torch


def test_temporal_ensemble_weights_and_sparse_queries():
    from noeira_b200.models.act_inference import TemporalEnsemble
    K, A, m = 4, 2, 0.5
    ens = TemporalEnsemble(A, K, m)
    chunks = {i: np.full((K, A), float(i + 1), dtype=np.float32) + np.arange(K, dtype=np.float32)[:, None] for i in range(6)}
    for t in range(6):
        ens.push(t, chunks[t])
        a = ens.action_at(t)
        i_min = max(t - K + 1, 0)
        qs = list(range(i_min, t + 1))
        w = np.array([math.exp(-m * (i - i_min)) for i in qs])
        w /= w.sum()
        want = sum(wi * chunks[i][t - i] for wi, i in zip(w, qs))
        assert np.allclose(a, want, atol=1e-6) and ens.n_contributors(t) == len(qs)
    # sparse: only steps 0 and 2 were queried → exponent is the age in grid steps
    ens.reset()
    ens.push(0, chunks[0])
    ens.push(2, chunks[2])
    a = ens.action_at(3)
    w = np.array([1.0, math.exp(-m * 2)])
    w /= w.sum()
    assert np.allclose(a, w[0] * chunks[0][3] + w[1] * chunks[2][1], atol=1e-6)
    ens.reset()
    try:
        ens.action_at(0)
        assert False
    except RuntimeError:
        pass


def test_act_norm_file_roundtrip_is_bit_exact(tmp_path):
    from noeira_b200.models.act_inference import ACTNorm, denormalize
    g = np.random.default_rng(0)
    q, a = g.normal(size=(50, 6)).astype(np.float32), g.normal(size=(50, 7, 6)).astype(np.float32)
    n = ACTNorm.from_data(q, a, cameras=["front", "wrist"], img_h=480, img_w=640, n_episodes=5, store="store.h5")
    p = str(tmp_path / "ck" / "norm.json")
    n.save(p)
    m = ACTNorm.load(p)
    for k in ("qpos_mean", "qpos_std", "action_mean", "action_std"):
        assert np.array_equal(np.float32(getattr(n, k)), np.float32(getattr(m, k)))
    assert m.cameras == ["front", "wrist"] and m.img_h == 480 and m.n_rows == 50
    lo, hi = m.action_box(0.05)
    assert (lo < np.asarray(m.action_min)).all() and (hi > np.asarray(m.action_max)).all()
    assert np.allclose(denormalize(np.zeros(6), m.action_mean, m.action_std), m.action_mean)


def test_act_policy_closed_loop_cpu():
    from noeira_b200.models.act import ACTConfig, ACTModel
    from noeira_b200.models.act_inference import ACTNorm, ACTPolicy
    cfg = ACTConfig(height=64, width=96, chunk=5, enc_layers=1, dec_layers=1, dim=64, heads=4, ff=128)
    model = ACTModel(cfg)
    model.train(False) if hasattr(model, "train") else None
    norm = ACTNorm.from_data(np.random.default_rng(1).normal(size=(20, 6)).astype(np.float32),
                             np.random.default_rng(2).normal(size=(20, 6)).astype(np.float32))
    pol = ACTPolicy(model, norm, query_every=2)
    img = torch.randint(0, 256, (cfg.n_cam, 3, cfg.height, cfg.width), dtype=torch.uint8)
    acts = [pol.act(np.zeros(6, np.float32), img) for _ in range(5)]
    assert all(a.shape == (6,) and np.isfinite(a).all() for a in acts)
    assert pol.ens.n_contributors(4) == 3            # queries at steps 0, 2, 4
    lo, hi = norm.action_box()
    assert all((a >= lo - 1e-6).all() and (a <= hi + 1e-6).all() for a in acts)
