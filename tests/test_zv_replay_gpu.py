"""Device replay kernels: ring store with wrap-around and demo prefix, uniform / ERE / PER sampling, gather."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rows(n, off, O=5, A=2):
    i = torch.arange(off, off + n, dtype=torch.float32, device="cuda")
    return (i[:, None] + torch.zeros(n, O, device="cuda"), -i[:, None] + torch.zeros(n, A, device="cuda"), i * 0.5,
            i[:, None] + 0.25 + torch.zeros(n, O, device="cuda"), (i % 7 == 0).float())


def test_ring_store_wraps_and_keeps_demo_prefix():
    from noeira_b200.data.replay import StoreReplayGpu
    rb = StoreReplayGpu(100, 5, 2, demo_prefix=10, per_alpha=0.0)
    rb.buf[:10, 0] = -1.0                                  # stands for demonstrations
    for k in range(8):
        rb.store_batch(*_rows(16, 16 * k))
    assert rb.size == 100 and int(rb.meta[0]) == 10 + (128 % 90)
    assert (rb.buf[:10, 0] == -1).all()
    vals = rb.buf[10:, 0].sort().values
    assert vals.tolist() == [float(v) for v in range(38, 128)]          # the newest 90 transitions survive
    idx, _ = rb.indices(4096, "uniform")
    assert idx.min() >= 0 and idx.max() < 100 and idx.unique().numel() > 90
    (s, a, r, sp, d), _, _ = rb.sample(64)
    on = s[:, 0] >= 0
    assert torch.allclose(sp[on, 0], s[on, 0] + 0.25) and torch.allclose(a[on, 0], -s[on, 0]) and torch.allclose(r[on], 0.5 * s[on, 0])
    i1, _ = rb.indices(256, "uniform")
    a1 = i1.clone()
    i2, _ = rb.indices(256, "uniform")
    assert not torch.equal(a1, i2)                         # the device counter advances the stream
    e, _ = rb.indices(2048, "ere", ere_frac=0.2, c_min=10)
    recent = rb.buf[e, 0]
    assert recent.min() >= 128 - 20 and recent.max() == 127    # only the most recent 20 = 0.2 x size transitions


def test_per_sum_tree_matches_priorities():
    from noeira_b200.data.replay import StoreReplayGpu
    rb = StoreReplayGpu(64, 5, 2, per_alpha=1.0, per_beta=0.5, seed=3)
    rb.store_batch(*_rows(64, 0))
    assert abs(float(rb.tree[1]) - 64.0) < 1e-3            # every new transition enters with priority 1
    pr = torch.zeros(64, device="cuda")
    pr[5], pr[17], pr[40] = 3.0, 1.0, 4.0
    rb.update_priorities(torch.arange(64, device="cuda"), pr)
    assert abs(float(rb.tree[1]) - 8.0) < 1e-3
    counts = torch.zeros(64, device="cuda")
    for _ in range(40):
        idx, w = rb.indices(256, "per")
        counts += torch.bincount(idx, minlength=64).float()
    frac = counts / counts.sum()
    assert abs(float(frac[5]) - 3 / 8) < 0.02 and abs(float(frac[17]) - 1 / 8) < 0.02 and abs(float(frac[40]) - 4 / 8) < 0.02
    idx, w = rb.indices(256, "per")
    assert w.max() == 1.0 and torch.allclose(w[idx == 17].mean() / w[idx == 40].mean(), torch.tensor(2.0, device="cuda"), rtol=1e-3)


def test_per_sum_tree_large_capacity():
    """Capacity above 2^19 leaves: the root must equal the sum of the leaves after a batched update, and uniform
    stores that never sample by priority must not touch the tree."""
    from noeira_b200.data.replay import StoreReplayGpu
    cap = (1 << 20) + 7
    rb = StoreReplayGpu(cap, 3, 1, per_alpha=1.0, seed=1)
    assert rb.leaves == 1 << 21
    g = torch.Generator(device="cuda").manual_seed(0)
    idx = torch.randint(0, cap, (50_000,), device="cuda", generator=g)
    pr = torch.rand(50_000, device="cuda", generator=g) + 0.1
    rb.update_priorities(idx, pr)
    leaves = rb.tree[rb.leaves:].double()
    assert abs(float(rb.tree[1]) - float(leaves.sum())) < 1e-3 * float(leaves.sum())
    # every inner node is the sum of its children
    inner = rb.tree[1: rb.leaves]
    kids = rb.tree[2: 2 * rb.leaves].view(-1, 2).sum(1)
    assert torch.allclose(inner, kids, rtol=1e-6, atol=1e-6)
    plain = StoreReplayGpu(1024, 3, 1, prioritized=False)
    plain.store_batch(torch.zeros(8, 3, device="cuda"), torch.zeros(8, 1, device="cuda"), torch.zeros(8, device="cuda"),
                      torch.zeros(8, 3, device="cuda"), torch.zeros(8, device="cuda"))
    assert plain.tree.numel() == 2 and float(plain.tree.sum()) == 0.0
