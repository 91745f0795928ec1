"""tcgen05 GEMM entry point (csrc/gemm_tcgen05.cu)."""
from __future__ import annotations

import ctypes

import torch

from .._native import check, cuda_lib, ptr, stream_ptr
from .status import device_status
from .streams import ws_key

ACT = {None: 0, "none": 0, "relu": 1, "tanh": 2, "gelu": 3, "silu": 4, "sigmoid": 5, "add": 16}

# Split-K workspace: [1024 u32 tile counters | fp32 partial tiles].  One per device, allocated on first use
# (its address is then stable, so captured CUDA graphs can replay).  GEMMs on ONE stream serialise and may
# share it; code inside an ``ops.streams.Branch`` gets the private workspace of that branch's slot.
WORKSPACE_BYTES = 4096 + (32 << 20)
_WS = {}


def new_workspace(device) -> torch.Tensor:
    return torch.zeros(WORKSPACE_BYTES, dtype=torch.uint8, device=device)


def default_workspace(device) -> torch.Tensor:
    key = ws_key(device)
    w = _WS.get(key)
    if w is None:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("run one eager GEMM on this device before capturing a CUDA graph")
        w = new_workspace(device)
        _WS[key] = w
    return w


TWO_CTA_AUTO, TWO_CTA_OFF, TWO_CTA_FORCE = 0, 1, 2


def set_two_cta_mode(mode: int) -> int:
    """Tile form of large GEMMs: by problem size (default), one-CTA tiles only, or 256 x 256 tiles computed by a pair
    of CTAs (``tcgen05.mma.cta_group::2``) whenever M, N >= 256.  Returns the previous setting."""
    return int(cuda_lib().nb_gemm_two_cta_mode(ctypes.c_int(mode)))


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, out: torch.Tensor = None,
         out_dtype=torch.bfloat16, accumulate: bool = False, alpha: float = 1.0, bias: torch.Tensor = None,
         act=None, aux: torch.Tensor = None, dact=None, bn: int = 0, n: int = None,
         workspace: torch.Tensor = None, residual: torch.Tensor = None) -> torch.Tensor:
    """``out[M,N] = epi(alpha · A·B)`` in bf16 with fp32 accumulation; fp32 operands run as TF32 (``kind::tf32``: the
    copy into shared memory rounds them to a 10-bit mantissa, accumulation and the default output stay fp32).

    ``a`` is ``[M,K]`` (``a_mn=False``) or ``[K,M]`` (``a_mn=True``); ``b`` is ``[N,K]`` (``b_mn=False``) or
    ``[K,N]`` (``b_mn=True``).  Rows may be strided (pitch a multiple of 8 elements).  ``bias`` fp32 ``[N]``;
    ``act`` applied after the bias; ``dact`` multiplies by the derivative of that activation evaluated on the
    saved bf16 tensor ``aux [M,N]`` (output for tanh/relu/sigmoid, input for gelu/silu); ``accumulate`` adds
    into an fp32 ``out``; ``residual`` (bf16 ``[M,N]``, exclusive with ``dact``) is added after the activation.
    """
    if residual is not None:
        assert dact is None and aux is None
        aux, dact = residual, "add"
    tf32 = a.dtype == torch.float32
    assert a.dtype == b.dtype and a.dtype in (torch.bfloat16, torch.float32)
    assert a.stride(-1) == 1 and b.stride(-1) == 1
    if tf32 and out is None and out_dtype == torch.bfloat16:
        out_dtype = torch.float32
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    assert Kb == K, (a.shape, b.shape, a_mn, b_mn)
    if n is not None:
        N = n
    if out is None:
        out = torch.empty(M, N, device=a.device, dtype=out_dtype)
    assert out.stride(-1) == 1 and out.shape[0] == M
    out_f32 = out.dtype == torch.float32
    assert out_f32 or out.dtype == torch.bfloat16
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() >= N
    if aux is not None:
        assert aux.dtype == torch.bfloat16 and aux.stride(-1) == 1
    st = device_status(a.device)
    ws = workspace if workspace is not None else default_workspace(a.device)
    rc = (cuda_lib().nb_gemm_tf32 if tf32 else cuda_lib().nb_gemm_bf16)(
        ptr(a), ptr(b), ptr(out), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
        ctypes.c_int(a.stride(0)), ctypes.c_int(b.stride(0)), ctypes.c_int(out.stride(0)),
        ctypes.c_int(int(a_mn)), ctypes.c_int(int(b_mn)), ctypes.c_int(int(out_f32)), ctypes.c_int(int(accumulate)),
        ctypes.c_float(alpha), ptr(bias), ctypes.c_int(ACT[act]), ptr(aux),
        ctypes.c_int(aux.stride(0) if aux is not None else 0), ctypes.c_int(ACT[dact]), ptr(st), ctypes.c_int(bn),
        ptr(ws), ctypes.c_longlong(ws.numel()), stream_ptr())
    check(rc, "nb_gemm_tf32" if tf32 else "nb_gemm_bf16")
    return out
