"""Distributed gates on the in-process simulator (threads, rank-ordered reductions) and on gloo processes.
Modelled on the reference's gates (tests/nn/distributed/test_fibers.mojo, test_ddp_mlp.mojo, test_zero1.mojo):
N=1 identity bit-exact, replica agreement bit-exact, DDP vs ZeRO bit-exact without clip, a failing rank or a
missing rendezvous ends the run with an error instead of a hang."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _net():
    from noeira_b200 import nn
    nn.manual_seed(5)
    return nn.Sequential(nn.LinearTanh(12, 40), nn.LinearTanh(40, 40), nn.Linear(40, 3))


def _train(comm, strategy, steps=4, clip=0.0, world_batch=16):
    from noeira_b200 import nn
    from noeira_b200.parallel.strategy import STRATEGIES
    net = _net()
    opt = nn.AdamW(net.named_params(), lr=1e-2, weight_decay=0.01)
    st = STRATEGIES[strategy](opt, comm, model=net)
    st.sync_params()
    g = torch.Generator().manual_seed(0)
    per = world_batch // comm.world
    peak = 0
    for _ in range(steps):
        x = torch.randn(world_batch, 12, generator=g)
        y = torch.randn(world_batch, 3, generator=g)
        xs, ys = x[comm.rank * per:(comm.rank + 1) * per], y[comm.rank * per:(comm.rank + 1) * per]
        st.begin_step()
        out = net.forward(xs)
        net.vjp(2.0 * (out - ys) / per)
        st.reduce_grads()
        if clip > 0:
            st.clip_grads(clip)
        st.step()
        peak = max(peak, st.state_bytes_per_rank())
    return st.full_values(), st.state_bytes_per_rank()


def test_n1_identity_and_replica_agreement_and_strategy_equivalence():
    from noeira_b200.parallel.fibers import run_ranks
    base = run_ranks(1, lambda c: _train(c, "ddp"))[0][0]
    single = _train(type("C", (), dict(world=1, rank=0, all_reduce=lambda s, t: None, broadcast=lambda s, t, src=0: None))(), "ddp")[0]
    assert torch.equal(base, single)                                   # N=1 identity, bit exact
    res = {}
    for strat in ("ddp", "zero1", "zero2", "zero3"):
        out = run_ranks(2, lambda c, s=strat: _train(c, s))
        assert torch.equal(out[0][0], out[1][0]), strat                # replicas agree bit for bit
        res[strat] = out[0]
    for strat in ("zero1", "zero2", "zero3"):
        assert torch.equal(res["ddp"][0], res[strat][0]), strat        # DDP == ZeRO without clip
    # bytes actually allocated between steps: DDP 4Ψ, ZeRO-1 2Ψ + 3Ψ/N, ZeRO-2 Ψ + 3Ψ/N, ZeRO-3 4Ψ/N (N = 2)
    psi = res["ddp"][1] / 4
    assert res["ddp"][1] > res["zero1"][1] > res["zero2"][1] > res["zero3"][1]
    assert res["zero1"][1] <= 3.6 * psi and res["zero2"][1] <= 2.6 * psi and res["zero3"][1] <= 2.1 * psi
    # two ranks with half batches ≈ one rank with the full batch (mean of shard means)
    assert torch.allclose(res["ddp"][0], base, atol=1e-5)


def test_clip_norm_matches_between_ddp_and_zero():
    from noeira_b200.parallel.fibers import run_ranks
    a = run_ranks(2, lambda c: _train(c, "ddp", clip=0.05))[0][0]
    b = run_ranks(2, lambda c: _train(c, "zero1", clip=0.05))[0][0]
    assert torch.allclose(a, b, atol=1e-6)


def test_rank_exception_ends_the_run_without_hanging():
    from noeira_b200.parallel.fibers import run_ranks

    def body(c):
        t = torch.ones(4)
        c.all_reduce(t)
        if c.rank == 1:
            raise ValueError("rank 1 broke")
        c.all_reduce(t)
        return t

    with pytest.raises(ValueError, match="rank 1 broke"):
        run_ranks(3, body, timeout=5)


def test_missing_rendezvous_is_an_error_not_a_hang():
    from noeira_b200.parallel.fibers import CollectiveMismatch, RankFailed, run_ranks

    def body(c):
        t = torch.ones(2)
        c.all_reduce(t)
        if c.rank != 0:
            c.all_reduce(t)       # rank 0 never joins this one
        return t

    with pytest.raises((RankFailed, CollectiveMismatch)):
        run_ranks(2, body, timeout=5)

    def body2(c):
        t = torch.ones(2)
        if c.rank == 0:
            c.all_reduce(t)
        else:
            c.barrier()
        return t

    with pytest.raises((RankFailed, CollectiveMismatch)):
        run_ranks(2, body2, timeout=5)


def test_collectives_are_rank_ordered_and_deterministic():
    from noeira_b200.parallel.fibers import run_ranks

    def body(c):
        t = torch.full((3,), 0.1 * (c.rank + 1))
        c.all_reduce(t)
        out = torch.zeros(2)
        c.reduce_scatter(out, torch.arange(8.0) + c.rank)
        gat = torch.zeros(8)
        c.all_gather(gat, torch.full((2,), float(c.rank)))
        return t, out, gat

    r = run_ranks(4, body)
    exp = ((torch.tensor(0.1) + torch.tensor(0.2)) + torch.tensor(0.3)) + torch.tensor(0.4)
    assert all(torch.equal(x[0], torch.full((3,), float(exp))) for x in r)
    assert torch.equal(r[1][1], torch.tensor([4 * 2.0 + 6, 4 * 3.0 + 6]))
    assert torch.equal(r[2][2], torch.tensor([0., 0, 1, 1, 2, 2, 3, 3]))


@pytest.mark.parametrize("strategy", ["ddp", "ddp_overlap"])
def test_gloo_processes_match_simulator(strategy):
    """Two real processes over gloo reproduce the simulator's DDP result bit for bit (also with the asynchronous,
    bucketed reduction of the overlapped strategy)."""
    from noeira_b200.parallel.fibers import run_ranks
    sim = run_ranks(2, lambda c: _train(c, "ddp"))[0][0]
    import tempfile
    with tempfile.TemporaryDirectory() as d:
        env = dict(os.environ, OUT=os.path.join(d, "v"), OMP_NUM_THREADS="1", STRATEGY=strategy)
        r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                            "--master-addr", "127.0.0.1", "--master-port", "29731",
                            os.path.join(ROOT, "tests", "mp", "gloo_worker.py")], env=env, capture_output=True, text=True,
                           timeout=240)
        assert r.returncode == 0, r.stderr[-2000:]
        v0, v1 = torch.load(os.path.join(d, "v0")), torch.load(os.path.join(d, "v1"))
    assert torch.equal(v0, v1)
    assert torch.equal(v0, sim)


def test_zero3_units_are_gathered_only_around_their_own_forward_and_backward():
    from noeira_b200 import nn
    from noeira_b200.parallel.fibers import run_ranks
    from noeira_b200.parallel.strategy import Zero3

    def body(c):
        net = _net()
        opt = nn.AdamW(net.named_params(), lr=1e-2)
        seen, box = [], []
        for i, child in enumerate(net.mods):         # recorders go in first, so the strategy's hooks wrap them
            f = child.forward
            child.forward = (lambda f, i: lambda *a, **k: (seen.append((i, [u["live_v"] for u in box[0].units])), f(*a, **k))[1])(f, i)
        st = Zero3(opt, c, model=net)
        box.append(st)
        assert st.hooked and len(st.units) == 3
        st.sync_params()
        x = torch.randn(4, 12)
        st.begin_step()
        out = net.forward(x)
        live_during = [s[1] for s in seen]
        net.vjp(out)
        st.reduce_grads()
        st.step()
        idle = [(u["live_v"], u["live_g"]) for u in st.units]
        return live_during, idle, st.state_bytes_per_rank(), opt.arena.numel

    for live_during, idle, nbytes, numel in run_ranks(2, body):
        # when unit i's own forward runs, exactly unit i is materialised
        assert live_during == [[True, False, False], [False, True, False], [False, False, True]]
        assert idle == [(False, False)] * 3
        assert nbytes <= 4 * 4 * numel / 2 * 1.1          # values, gradients and both moments: a shard of each


def test_overlapped_ddp_reduces_buckets_during_backward_and_matches_ddp():
    """The bucketed reducer is driven by the model's own backward: with a small bucket size every unit is its own bucket,
    the buckets of the later units go out while the backward is still running, and the result is bit-identical to the
    reduce-after-backward strategy."""
    from noeira_b200 import nn
    from noeira_b200.parallel.fibers import run_ranks
    from noeira_b200.parallel.strategy import OverlappedDataParallel

    def body(comm):
        net = _net()
        opt = nn.AdamW(net.named_params(), lr=1e-2, weight_decay=0.01)
        st = OverlappedDataParallel(opt, comm, model=net, bucket_bytes=64)
        st.sync_params()
        g = torch.Generator().manual_seed(0)
        per = 16 // comm.world
        for _ in range(4):
            x = torch.randn(16, 12, generator=g)
            y = torch.randn(16, 3, generator=g)
            xs, ys = x[comm.rank * per:(comm.rank + 1) * per], y[comm.rank * per:(comm.rank + 1) * per]
            out = net.forward(xs)
            net.vjp(2.0 * (out - ys) / per)
            st.reduce_grads()
            st.step()
        return st.full_values(), len(st.buckets), st.launched_during_backward, list(st.reducer.order)

    out = run_ranks(2, body)
    ref = run_ranks(2, lambda c: _train(c, "ddp"))
    assert torch.equal(out[0][0], ref[0][0]) and torch.equal(out[0][0], out[1][0])
    vals, nb, during, order = out[0]
    assert nb == 3 and during == 4 * 3                       # every bucket of every step left from inside the backward
    assert order[0][0] > order[1][0] > order[2][0]           # last unit of the arena first
    default = run_ranks(2, lambda c: _train(c, "ddp_overlap"))
    assert torch.equal(default[0][0], ref[0][0])             # one 8 MB bucket: reduced by reduce_grads, same values
