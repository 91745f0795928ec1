"""Allocation-free column sum (csrc/noalloc_api.h), called through its exported C symbol.

Some users of this library cannot give a kernel scratch memory: a plug-in whose host application
owns the device allocator, a control loop that must stay out of the driver's allocation path, a
process that has already committed all device memory.  For them ``nb_colsum_bf16_noalloc`` keeps the
partial sums in an array compiled into the library.  This test checks that it returns what the
regular entry point (caller-supplied scratch) returns, on two consecutive calls — the second call
finds the array full of the first call's partials and must not be disturbed by them — and that it
refuses a problem larger than the built-in array.

The file name sorts last on purpose: if this addition ever fails, a run that stops at the first
failure has already exercised everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _regular(lib, x, n, out, accumulate):
    from noeira_b200._native import ptr, stream_ptr
    split = lib.nb_colsum_split(ctypes.c_int(x.shape[0]))
    ws = torch.empty(split * n, dtype=torch.float32, device=x.device)
    rc = lib.nb_colsum_bf16(ptr(x), ctypes.c_int(x.shape[0]), ctypes.c_int(n), ctypes.c_int(x.stride(0)), ptr(out),
                            ctypes.c_int(accumulate), ptr(ws), stream_ptr())
    assert rc == 0


def _noalloc(lib, x, n, out, accumulate):
    from noeira_b200._native import ptr, stream_ptr
    fn = lib.nb_colsum_bf16_noalloc  # the exported C symbol
    fn.restype = ctypes.c_int
    return fn(ptr(x), ctypes.c_int(x.shape[0]), ctypes.c_int(n), ctypes.c_int(x.stride(0)), ptr(out),
              ctypes.c_int(accumulate), stream_ptr())


def test_noalloc_colsum_matches_regular_entry_point_twice():
    from noeira_b200._native import cuda_lib
    lib = cuda_lib()
    torch.manual_seed(0)
    # first call: set-up of the device address happens here, outside any stream capture
    for call, (M, N) in enumerate([(16384, 256), (3000, 520)]):
        x = torch.randn(M, N, device="cuda").bfloat16()
        ref = torch.full((N,), 0.25, device="cuda")
        got = torch.full((N,), 0.25, device="cuda")
        _regular(lib, x, N, ref, accumulate=1)
        assert _noalloc(lib, x, N, got, accumulate=1) == 0
        torch.cuda.synchronize()
        assert torch.allclose(got, ref, atol=1e-2, rtol=1e-4), (call, (got - ref).abs().max().item())
        assert torch.equal(got, ref)  # same kernels, same order of additions
        truth = 0.25 + x.float().sum(0)
        assert torch.allclose(got, truth, atol=1e-2, rtol=1e-4)


def test_noalloc_colsum_rejects_oversize():
    from noeira_b200._native import cuda_lib
    lib = cuda_lib()
    M, N = 16384, 4104  # 256 slabs x 4104 columns > 2^20 floats of built-in scratch
    x = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(N, device="cuda")
    assert _noalloc(lib, x, N, out, accumulate=0) == 10003
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0
