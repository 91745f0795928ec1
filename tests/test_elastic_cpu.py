"""Failure detection without any GPU fault: heartbeat / watchdog on the host, a rank that leaves between steps, and a
restart of the checkpoint under a smaller world size that follows the uninterrupted trajectory."""
import os
import subprocess
import sys
import time

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class _Store(dict):
    def set(self, k, v):
        self[k] = v

    def get(self, k):
        return self[k]


def test_heartbeat_detects_stale_and_departed_peers():
    from noeira_b200.parallel.elastic import Heartbeat, PeerLost
    store, now = _Store(), [100.0]
    hbs = [Heartbeat(store, r, 3, deadline_s=5.0, clock=lambda: now[0]) for r in range(3)]
    hbs[0].check()
    now[0] += 4.0
    hbs[0].beat()
    hbs[1].beat()
    now[0] += 3.0                       # rank 2 last beat 7 s ago
    with pytest.raises(PeerLost) as e:
        hbs[0].check()
    assert e.value.ranks == [2] and hbs[0].alive() == [0, 1]
    hbs[2].beat()
    hbs[1].leave()
    with pytest.raises(PeerLost) as e:
        hbs[0].check()
    assert e.value.ranks == [1] and "left" in e.value.why


def test_step_watchdog_turns_a_missed_deadline_into_an_error():
    from noeira_b200.parallel.elastic import StepTimeout, StepWatchdog
    fired = []
    wd = StepWatchdog(0.15, on_timeout=fired.append, poll_s=0.02)
    wd.begin_step()
    time.sleep(0.05)
    wd.end_step()                        # in time: nothing
    wd.begin_step()
    time.sleep(0.4)
    with pytest.raises(StepTimeout):
        wd.end_step()
    assert len(fired) == 1 and fired[0] > 0.15
    wd.begin_step()
    wd.end_step()                        # usable again
    wd.close()


def _launch(world, phase, env, port):
    e = dict(os.environ, PHASE=str(phase), OMP_NUM_THREADS="1", **env)
    return subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                           "--master-addr", "127.0.0.1", "--master-port", str(port),
                           os.path.join(ROOT, "tests", "mp", "elastic_worker.py")], env=e, capture_output=True, text=True, timeout=300)


def test_rank_leaves_between_steps_and_run_resumes_on_fewer_ranks(tmp_path):
    out, ckpt = str(tmp_path / "o"), str(tmp_path / "ck")
    env = dict(OUT=out, CKPT=ckpt, TOTAL_STEPS="6", LEAVE_AT="3")
    r = _launch(3, 1, env, 29741)
    assert r.returncode == 0, r.stderr[-2000:]
    res = [torch.load(f"{out}.p1.r{k}") for k in range(3)]
    assert res[2]["status"] == "left"
    assert res[0]["status"] == "peer_lost:[2]:3" and res[1]["status"] == "peer_lost:[2]:3"   # noticed before step 3's collective
    # resume on 2 ranks from the checkpoint, same global batch
    r = _launch(2, 2, env, 29742)
    assert r.returncode == 0, r.stderr[-2000:]
    resumed = [torch.load(f"{out}.p2.r{k}") for k in range(2)]
    assert resumed[0]["status"] == "done" and torch.equal(resumed[0]["val"], resumed[1]["val"])
    # uninterrupted single-process run of the same 6 steps
    sys.path.insert(0, os.path.join(ROOT, "tests", "mp"))
    import elastic_worker as ew
    net, opt = ew.build()
    for step in range(6):
        x, y = ew.batch(step)
        o = net.forward(x)
        net.vjp(2.0 * (o - y) / x.shape[0])
        opt.step(zero_grad=True)
    assert torch.allclose(resumed[0]["val"], opt.arena.val, atol=2e-6), (resumed[0]["val"] - opt.arena.val).abs().max()
