"""Adapter / quantisation slots on a model's linears; the asynchronous action-chunk worker."""
import threading
import time

import pytest
import torch


def test_lora_and_q4_slots_replace_linears_in_place():
    from noeira_b200 import nn
    nn.manual_seed(0)
    net = nn.Sequential(nn.Linear(32, 64), nn.TransformerBlock(64, 4, 128, norm="rms", ffn="swiglu"), nn.Linear(64, 32))
    x = torch.randn(2, 5, 32)
    y0 = net.forward(x).clone()
    n = nn.add_lora(net, rank=8, predicate=lambda path, lin: "1." in path)      # the block's linears only
    assert n >= 4
    names = [k for k, _ in net.named_params()]
    assert any(k.endswith("lora_A.weight") for k in names) and any(".base_layer.weight" in k for k in names)
    assert torch.allclose(net.forward(x), y0, atol=1e-6)                        # B starts at zero: same function
    trainable = [k for k, p in net.named_params() if not p.frozen]
    assert all(("lora_" in k) or k.startswith("0.") or k.startswith("2.") or "norm" in k or "gamma" in k for k in trainable), trainable
    net.vjp(torch.randn(2, 5, 32))
    lora_b = [p for k, p in net.named_params() if k.endswith("lora_B.weight")]
    assert all(p.grad.abs().sum() > 0 for p in lora_b)
    base = [p for k, p in net.named_params() if ".base_layer.weight" in k]
    assert all(p._grd is None or p.grad.abs().sum() == 0 for p in base)
    # Q4 slots on another copy, with and without adapters
    nn.manual_seed(0)
    net2 = nn.Sequential(nn.Linear(32, 64), nn.TransformerBlock(64, 4, 128, norm="rms", ffn="swiglu"), nn.Linear(64, 32))
    nq = nn.quantize_linears(net2, lora_rank=8)
    assert nq >= 5
    y2 = net2.forward(x)
    assert (y2 - y0).abs().max() < 0.25 * y0.abs().max() and not torch.equal(y2, y0)
    assert any(k.endswith("scales") for k, _ in net2.named_states())


def test_query_worker_answers_off_thread_and_keeps_only_the_newest_observation():
    from noeira_b200.models.vla_worker import ChunkCursor, VLAQueryWorker
    started, release = threading.Event(), threading.Event()
    calls = []

    def query(obs):
        calls.append(int(obs[0]))
        if len(calls) == 1:
            started.set()
            release.wait(5.0)
        return obs.float().repeat(6, 1) + torch.arange(6.0)[:, None]

    w = VLAQueryWorker(query)
    try:
        assert w.latest() is None
        s1 = w.submit(torch.tensor([10.0]))
        assert started.wait(5.0)
        s2, s3 = w.submit(torch.tensor([20.0])), w.submit(torch.tensor([30.0]))      # 20 is replaced while 10 is running
        t0 = time.monotonic()
        assert w.latest() is None and time.monotonic() - t0 < 0.05               # non-blocking read
        release.set()
        seq, chunk, secs = w.wait(newer_than=s1)
        assert seq == s3 and calls == [10, 30] and w.dropped == 1
        assert chunk.shape == (6, 1) and float(chunk[2]) == 32.0 and secs >= 0
        cur = ChunkCursor()
        cur.offer(chunk, observed_at_tick=100)
        assert float(cur.action(100)) == 30.0 and float(cur.action(103)) == 33.0 and float(cur.action(200)) == 35.0
        assert cur.remaining(103) == 2
        cur.offer(chunk + 100, observed_at_tick=102)                              # a newer chunk takes over mid-way
        assert float(cur.action(103)) == 131.0
    finally:
        w.close()


def test_query_worker_reports_a_failing_query():
    from noeira_b200.models.vla_worker import VLAQueryWorker

    def bad(obs):
        raise ValueError("camera unplugged")

    w = VLAQueryWorker(bad)
    try:
        w.submit(torch.zeros(1))
        with pytest.raises(RuntimeError):
            w.wait(timeout=5.0)
        assert isinstance(w.error, ValueError)
    finally:
        w.close()
