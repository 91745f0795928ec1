import gzip
import struct

import numpy as np


def test_idx_cifar_charcorpus(tmp_path):
    from noeira_b200.data.datasets import CharCorpus, load_cifar10_bin, load_mnist_idx
    imgs = np.random.default_rng(0).integers(0, 256, (10, 28, 28), dtype=np.uint8)
    labels = np.arange(10, dtype=np.uint8)
    (tmp_path / "im.gz").write_bytes(gzip.compress(struct.pack(">IIII", 2051, 10, 28, 28) + imgs.tobytes()))
    (tmp_path / "lb").write_bytes(struct.pack(">II", 2049, 10) + labels.tobytes())
    x, y = load_mnist_idx(str(tmp_path / "im.gz"), str(tmp_path / "lb"))
    assert np.array_equal(x, imgs) and np.array_equal(y, labels)
    rec = np.random.default_rng(1).integers(0, 256, (7, 3073), dtype=np.uint8)
    (tmp_path / "b1.bin").write_bytes(rec.tobytes())
    cx, cy = load_cifar10_bin([str(tmp_path / "b1.bin")])
    assert cx.shape == (7, 3, 32, 32) and np.array_equal(cy, rec[:, 0]) and cx[3, 2, 31, 31] == rec[3, -1]
    c = CharCorpus("hello world")
    assert c.vocab == 8 and c.decode(c.encode("low")) == "low" and len(c.tokens) == 11


def test_trajectory_store_and_loader(tmp_path):
    from noeira_b200.data.datasets import TrajectoryStore, TrajectoryWriter
    w = TrajectoryWriter(str(tmp_path / "t.traj"), {"obs": 3, "act": 2, "rew": 1}, {"env": "test"})
    rng = np.random.default_rng(0)
    eps = []
    for T in (5, 17, 40):
        e = dict(obs=rng.normal(size=(T, 3)), act=rng.normal(size=(T, 2)), rew=rng.normal(size=(T,)))
        eps.append(e)
        w.add_episode(**e)
    w.close()
    s = TrajectoryStore(str(tmp_path / "t.traj"))
    assert s.lengths == [5, 17, 40] and s.n_steps == 62 and s.meta == {"env": "test"} and s.width == 6
    assert np.allclose(s.episode(1)["act"], eps[1]["act"].astype(np.float32))
    allv = s.all_steps()
    assert np.allclose(allv["rew"][:5, 0], eps[0]["rew"].astype(np.float32))
    it = s.loader(batch=16, seed=1)
    seen = []
    for batch, idx in it:
        assert np.allclose(batch["obs"], allv["obs"][idx.astype(np.int64)])
        seen.extend(idx.tolist())
    assert len(seen) == 48 and len(set(seen)) == 48          # drop_last: 3 full batches of distinct steps
    it.close()


def test_hyperparam_search(tmp_path):
    from noeira_b200.core import hyperparam as hp
    g = hp.grid({"lr": [1e-3, 1e-2], "h": [32, 64, 128]})
    assert len(g) == 6 and {"lr": 1e-2, "h": 64} in g
    r = hp.random_configs({"lr": ("loguniform", 1e-5, 1e-1), "layers": ("int", 1, 4), "act": ["relu", "tanh"]}, 20, seed=3)
    assert len(r) == 20 and all(1e-5 <= c["lr"] <= 1e-1 and 1 <= c["layers"] <= 4 for c in r)
    assert r == hp.random_configs({"lr": ("loguniform", 1e-5, 1e-1), "layers": ("int", 1, 4), "act": ["relu", "tanh"]}, 20, seed=3)
    rows = hp.search(g, lambda c: -abs(c["lr"] - 1e-2) - abs(c["h"] - 64) / 1000, csv_path=str(tmp_path / "s.csv"))
    assert rows[0]["lr"] == 1e-2 and rows[0]["h"] == 64
    assert open(tmp_path / "s.csv").read().splitlines()[0] == "lr,h,score"


def test_successive_halving_and_tabular_search(tmp_path):
    from noeira_b200.agents.tabular import GridWorld, TabularAgent
    from noeira_b200.core import hyperparam as hp
    calls = []

    def objective(cfg, budget):                       # better configurations improve faster with budget
        calls.append((cfg["q"], budget))
        return cfg["q"] * (1 - 0.5 ** budget)

    rows = hp.successive_halving([{"q": q} for q in range(9)], objective, min_budget=1, eta=3, max_budget=9,
                                 csv_path=str(tmp_path / "sh.csv"))
    assert rows[0]["q"] == 8 and rows[0]["budget"] == 9 and rows[0]["rung"] == 2
    assert sorted(b for _, b in calls) == [1] * 9 + [3] * 3 + [9]           # 9 → 3 → 1 survivors
    assert open(tmp_path / "sh.csv").read().splitlines()[0] == "q,budget,score,rung"
    res = hp.search_tabular(lambda c: TabularAgent(25, 4, kind=c["kind"], alpha=c["alpha"], eps=0.1, seed=0), lambda: GridWorld(),
                            {"kind": ["q_learning", "sarsa"], "alpha": [0.02, 0.3]}, episodes=150)
    assert len(res) == 4 and res[0]["score"] >= res[-1]["score"] and res[0]["score"] > 0.5 and {r["kind"] for r in res} == {"q_learning", "sarsa"}


def test_act_dataset_chunks_and_masks():
    import torch
    from noeira_b200.data.act_dataset import ACTDataset, synthetic_episodes
    eps = synthetic_episodes(4, 30, cams=2, height=8, width=10, seed=1)
    ds = ACTDataset(eps, chunk=12, seed=0)
    assert ds.n_steps == sum(e["qpos"].shape[0] for e in eps)
    q, img, act, valid = ds.sample(256)
    assert q.shape == (256, 6) and img.shape == (256, 2, 3, 8, 10) and img.dtype == torch.uint8
    assert act.shape == (256, 12, 6) and valid.shape == (256, 14) and (valid[:, :2] == 1).all()
    # padded steps are exactly zero and masked; real steps reproduce the episode's actions
    assert (act[valid[:, 2:] == 0] == 0).all() and (valid[:, 2:].sum(1) >= 1).all() and (valid[:, 2:].sum(1) < 12).any()
    ds.gen.manual_seed(0)
    t = torch.randint(0, ds.n_steps, (256,), generator=ds.gen)
    k = int((valid[:, 2:].sum(1) == 12).nonzero()[0])
    assert torch.allclose(ds.denormalise_action(act[k]), ds.action[t[k]: t[k] + 12], atol=1e-5)
    m = valid[:, 2:].bool()
    assert (valid[:, 2:].cumsum(1)[~m] == valid[:, 2:].sum(1, keepdim=True).expand(-1, 12)[~m]).all()   # padding only at the end


def test_zstd_stream_and_tar(tmp_path):
    import os
    from noeira_b200.io import formats as F
    data = (b"trajectory " * 5000) + os.urandom(3000)
    z = F.zstd_compress(data, 5)
    assert len(z) < len(data) // 4 and F.zstd_decompress(z) == data
    two = z + F.zstd_compress(b"second frame")
    assert F.zstd_decompress(two, chunk=1024) == data + b"second frame"        # concatenated frames, small output window
    import pytest
    with pytest.raises(ValueError):
        F.zstd_decompress(z[:-5])
    p = str(tmp_path / "shard.tar.gz")
    F.write_tar(p, {"a/x.npy": b"123", "a/y.json": b"{}", "b/z.bin": bytes(range(10))}, compression="gz")
    assert F.read_tar(p) == {"a/x.npy": b"123", "a/y.json": b"{}", "b/z.bin": bytes(range(10))}
    assert list(F.read_tar(p, prefix="b/")) == ["b/z.bin"]
