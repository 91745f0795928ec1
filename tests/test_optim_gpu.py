import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_arena_adamw_matches_torch():
    from noeira_b200._native import check, cuda_lib, ptr, stream_ptr
    lib = cuda_lib()
    torch.manual_seed(0)
    n = 32 * 1000
    val = torch.randn(n, device="cuda")
    grd = torch.randn(n, device="cuda")
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    shadow = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    flags = torch.ones(n // 32, device="cuda", dtype=torch.uint8)
    flags[::3] = 0  # no decay rows
    p = torch.nn.Parameter(val.clone())
    hyper = torch.zeros(16, device="cuda")
    hyper[:5] = torch.tensor([1e-2, 0.9, 0.999, 1e-8, 0.1])
    hyper[5:9] = torch.tensor([0.0, 1.0, 1.0, 0.5])
    decay = flags.bool().repeat_interleave(32)
    ref = val.clone()
    rm, rv = torch.zeros_like(ref), torch.zeros_like(ref)
    for t in range(1, 4):
        check(lib.nb_adam_advance(ptr(hyper), stream_ptr()), "advance")
        check(lib.nb_arena_adamw(ptr(val), ptr(grd), ptr(m), ptr(v), ptr(shadow), ptr(flags), ctypes.c_longlong(n),
                                 ptr(hyper), ctypes.c_int(0), stream_ptr()), "adamw")
        g = grd * 0.5
        rm = 0.9 * rm + 0.1 * g
        rv = 0.999 * rv + 0.001 * g * g
        upd = (rm / (1 - 0.9 ** t)) / ((rv / (1 - 0.999 ** t)).sqrt() + 1e-8)
        upd = upd + torch.where(decay, 0.1 * ref, torch.zeros_like(ref))
        ref = ref - 1e-2 * upd
    torch.cuda.synchronize()
    assert torch.allclose(val, ref, atol=1e-5, rtol=1e-5)
    assert torch.allclose(shadow.float(), val, atol=1e-2, rtol=1e-2)
    assert p is not None


def test_sumsq_clip_polyak():
    from noeira_b200._native import check, cuda_lib, ptr, stream_ptr
    lib = cuda_lib()
    n = 4 * 100003 - 4 * 100003 % 4
    g = torch.randn(n, device="cuda")
    partials = torch.zeros(2048, device="cuda")
    ticket = torch.zeros(1, device="cuda", dtype=torch.int32)
    out = torch.zeros(1, device="cuda")
    for _ in range(2):
        check(lib.nb_arena_sumsq(ptr(g), ctypes.c_longlong(n), ptr(partials), ptr(ticket), ptr(out), stream_ptr()), "sumsq")
    torch.cuda.synchronize()
    assert abs(out.item() - (g.double() ** 2).sum().item()) / n < 1e-4
    hyper = torch.zeros(16, device="cuda")
    norm = torch.zeros(1, device="cuda")
    check(lib.nb_clip_finalize(ptr(out), ctypes.c_float(1.0), ctypes.c_float(1.0), ptr(hyper), ptr(norm), stream_ptr()), "clip")
    torch.cuda.synchronize()
    assert abs(hyper[8].item() - 1.0 / (g.norm().item() + 1e-6)) < 1e-6
    a, b = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
    ref = a + 0.005 * (b - a)
    check(lib.nb_polyak(ptr(a), ptr(b), ctypes.c_longlong(n), ctypes.c_float(0.005), stream_ptr()), "polyak")
    torch.cuda.synchronize()
    assert torch.allclose(a, ref, atol=1e-6)


def test_step_many_equals_separate_steps():
    """Two optimizers stepped by the one-launch multi-arena kernel (step counters advanced inside it) against stepping
    each on its own: same step counters bit for bit, same values to rounding (the two kernels contract their
    multiply-adds differently, so the last bit of an update may differ)."""
    import torch
    from noeira_b200 import nn
    from noeira_b200.nn.optim import step_many
    nn.manual_seed(3)
    mk = lambda o: nn.Sequential(nn.LinearTanh(17, 256), nn.Linear(256, o)).to("cuda")
    a, b = [mk(6), mk(1)], [mk(6), mk(1)]
    for x, y in zip(a, b):
        y.copy_from(x)
    oa = [nn.AdamW(n.named_params(), lr=1e-2, weight_decay=0.01) for n in a]
    ob = [nn.AdamW(n.named_params(), lr=1e-2, weight_decay=0.01) for n in b]
    g = torch.Generator(device="cuda").manual_seed(0)
    for _ in range(3):
        for o1, o2 in zip(oa, ob):
            gr = torch.randn(o1.arena.numel, device="cuda", generator=g)
            o1.arena.grd.copy_(gr)
            o2.arena.grd.copy_(gr)
        step_many(oa, zero_grad=True)
        for o in ob:
            o.step(zero_grad=True)
    torch.cuda.synchronize()
    for o1, o2 in zip(oa, ob):
        assert torch.allclose(o1.arena.val, o2.arena.val, rtol=1e-5, atol=1e-7)
        assert torch.allclose(o1.arena.shadow.float(), o2.arena.shadow.float(), rtol=1e-2, atol=1e-6)
        assert torch.equal(o1.hyper, o2.hyper) and float(o1.arena.grd.abs().max()) == 0.0
