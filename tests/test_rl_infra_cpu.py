"""Shared RL infrastructure: running statistics, episode bookkeeping, cadence, generic drivers (CPU)."""
import numpy as np
import torch


def test_running_mean_std_matches_batch_statistics_and_skips_rows(tmp_path):
    from noeira_b200.training.rl import RunningMeanStd, norm_reward
    g = torch.Generator().manual_seed(0)
    rms = RunningMeanStd(3)
    chunks = [torch.randn(50, 3, generator=g) * 2 + 1 for _ in range(6)]
    for c in chunks:
        rms.update(c)
    allx = torch.cat(chunks).double()
    assert torch.allclose(rms.mean, allx.mean(0), atol=1e-3)
    assert torch.allclose(rms.var, allx.var(0, unbiased=False), atol=2e-3)
    # skipped rows do not count
    a, b = RunningMeanStd(3), RunningMeanStd(3)
    x = torch.randn(20, 3, generator=g)
    skip = torch.zeros(20, dtype=torch.bool)
    skip[::3] = True
    a.update(x, skip)
    b.update(x[~skip])
    assert torch.allclose(a.mean, b.mean) and torch.allclose(a.var, b.var) and torch.allclose(a.count, b.count)
    a.update(x, torch.ones(20, dtype=torch.bool))          # nothing left: unchanged
    assert torch.allclose(a.mean, b.mean) and torch.allclose(a.count, b.count)
    y = rms.normalize(chunks[0], clip=1.5)
    assert float(y.abs().max()) <= 1.5
    p = str(tmp_path / "obs_norm.txt")
    rms.save(p)
    assert open(p).read().split("\n")[0].startswith("count ")
    r2 = RunningMeanStd(3)
    r2.load(p)
    assert torch.allclose(r2.mean, rms.mean) and torch.allclose(r2.var, rms.var) and torch.allclose(r2.count, rms.count)
    assert float(norm_reward(torch.tensor([100.0]), torch.tensor(4.0), 10.0)) == 10.0
    assert abs(float(norm_reward(torch.tensor([1.0]), torch.tensor(4.0), 10.0)) - 0.5) < 1e-6


def test_episode_tracker_ring_and_cadence():
    from noeira_b200.training.rl import Cadence, DeviceMeanAccum, EpisodeReturnRing, EpisodeTracker
    t = EpisodeTracker(4, initial_fill=-10.0)
    assert t.mean_return() == -10.0
    t.add_reward(1.0)
    t.add_reward(2.0)
    t.end_episode()
    t.add_complete_return(5.0)
    assert t.ep_count == 2 and abs(t.mean_return() - (3 + 5 - 20) / 4) < 1e-9
    ring = EpisodeReturnRing(8, sync_every=2)
    tr = EpisodeTracker(100)
    ring.push(torch.tensor([1.0, 2.0, 3.0, 4.0]), torch.tensor([0.0, 1.0, 0.0, 1.0]))
    assert not ring.due()
    ring.push(torch.tensor([9.0, 8.0, 7.0, 6.0]), torch.tensor([1.0, 0.0, 0.0, 0.0]))
    assert ring.due() and ring.drain(tr) == 3
    assert sorted(tr.window[:3]) == [2.0, 4.0, 9.0] and tr.ep_count == 3
    assert ring.drain(tr) == 0
    c = Cadence(100)
    fired = [s for s in range(0, 1000, 64) if c(s)]
    assert fired == [128, 256, 320, 448, 512, 640, 704, 832, 960] or len(fired) == 9
    acc = DeviceMeanAccum(["loss", "kl"])
    acc.add("loss", torch.tensor(2.0))
    acc.add("loss", torch.tensor(4.0))
    out = acc.read()
    assert out["loss"] == 3.0 and np.isnan(out["kl"])


def test_offpolicy_driver_runs_sac_on_pendulum(tmp_path):
    from noeira_b200.agents.sac import SACConfig, SACTrainer
    from noeira_b200.data.replay import StoreReplay
    from noeira_b200.envs.classic import PendulumEnv
    from noeira_b200.training.rl import run_offpolicy_train_batched
    env = PendulumEnv(8, seed=0)
    env.max_steps = 25
    agent = SACTrainer(SACConfig(obs_dim=env.obs_dim, act_dim=env.act_dim, hidden=32, batch=32, seed=0))
    replay = StoreReplay(4096, env.obs_dim, env.act_dim, seed=0)
    rows = []

    class L:
        def log_scalars(self, step, d):
            rows.append((step, d))
    ck = str(tmp_path / "sac.ckpt")
    log = run_offpolicy_train_batched(agent, env, replay, 640, learning_starts=128, utd=1, batch_size=32, print_every=200,
                                      logger=L(), checkpoint_every=320, checkpoint_path=ck, episode_sync_every=4)
    assert agent.total_train_steps == (640 - 128) // 8 + 1
    assert log.episodes == 8 * (80 // 25) and len(log.steps) >= 3 and log.steps[-1] == 640
    assert rows and "mean_return" in rows[-1][1] and "critic_loss" in rows[-1][1]
    assert abs(log.mean_returns[-1]) > 0 and np.isfinite(log.mean_returns[-1])
    import os
    assert os.path.exists(ck)


def test_onpolicy_driver_stepwise_interface():
    from noeira_b200.envs.classic import PendulumEnv
    from noeira_b200.training.rl import run_onpolicy_train_batched

    class Stub:
        def __init__(self):
            self.recorded, self.updates = 0, 0

        def select_action_batched(self, obs):
            return torch.zeros(obs.shape[0], 1)

        def record_batch(self, obs, action, reward, next_obs, done, terminated):
            assert obs.shape == next_obs.shape and reward.shape == done.shape
            self.recorded += obs.shape[0]

        def train_step(self):
            if self.recorded % 64 == 0:
                self.updates += 1
                return {"loss": 0.0}
            return None

        def save(self, path):
            pass
    env = PendulumEnv(4, seed=1)
    env.max_steps = 10
    st = Stub()
    log = run_onpolicy_train_batched(st, env, 256, print_every=64, episode_sync_every=2)
    assert st.recorded == 256 and st.updates == 4 and log.episodes == 4 * (64 // 10)
    assert log.steps == [64, 128, 192, 256]
