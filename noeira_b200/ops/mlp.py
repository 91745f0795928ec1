"""Fused three-layer MLP forward (``csrc/mlp_fused_tcgen05.cu``): one launch for Linear+act → Linear+act → Linear with
hidden width 256, input width <= 64 and output width <= 16 — the actor / critic shape of the RL trainers."""
from __future__ import annotations

import ctypes

import torch

from .._native import check, cuda_lib, ptr, stream_ptr
from .gemm import ACT
from .status import device_status


def fusable(l1, l2, l3) -> bool:
    return (l1.on_cuda and l1.out_dim == 256 and l2.in_dim == 256 and l2.out_dim == 256 and l3.in_dim == 256
            and l1.in_dim <= 64 and l3.out_dim <= 16 and l1.act == l2.act and l1.act in ("tanh", "relu") and l3.act is None
            and l1.bias is not None and l2.bias is not None)


def mlp3_forward(x: torch.Tensor, l1, l2, l3, save: bool = True) -> torch.Tensor:
    """``x``: bf16 ``[M, >= in_dim]`` with a 16-byte row pitch.  Returns fp32 ``[M, out_dim]``.  With ``save`` the
    layers' backward caches (``_x`` / ``_saved``) are filled exactly as their own ``forward`` would, so the usual
    ``vjp`` chain runs unchanged."""
    M = x.shape[0]
    xv = x[:, : l1.in_dim]
    out = torch.empty(M, 16, device=x.device, dtype=torch.float32)
    h1 = torch.empty(M, 256, device=x.device, dtype=torch.bfloat16) if save else None
    h2 = torch.empty(M, 256, device=x.device, dtype=torch.bfloat16) if save else None
    w1, w2, w3 = l1.weight.shadow, l2.weight.shadow, l3.weight.shadow
    c = ctypes
    check(cuda_lib().nb_mlp3_fwd(ptr(xv), c.c_int(x.stride(0)), ptr(w1), c.c_int(w1.stride(0)), ptr(w2), c.c_int(w2.stride(0)),
                                 ptr(w3), c.c_int(w3.stride(0)), ptr(l1.bias.storage), ptr(l2.bias.storage),
                                 ptr(l3.bias.storage if l3.bias is not None else None), ptr(out), c.c_int(16), ptr(h1), ptr(h2),
                                 c.c_int(256), c.c_int(M), c.c_int(l1.in_dim), c.c_int(l3.out_dim), c.c_int(ACT[l1.act]),
                                 ptr(device_status(x.device)), stream_ptr()), "mlp3_fwd")
    y = out[:, : l3.out_dim]
    if save:
        for lin, xin, saved in ((l1, xv, h1), (l2, h1, h2), (l3, h2, y)):
            lin._lead = (M,)
            lin._x = xin
            lin._saved = saved
    return y
