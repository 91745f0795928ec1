"""Flash attention entry points (csrc/attention_tcgen05.cu) and the fp32 reference used by tests / CPU."""
from __future__ import annotations

import ctypes
import math

import torch

from .._native import check, cuda_lib, ptr, stream_ptr
from .status import device_status

MASK = {None: 0, "none": 0, "causal": 1, "block_causal": 2}


def attention_reference(q, k, v, scale=None, mask=None, frame=0, causal_off=0, key_valid=None, bias=None):
    """fp32 math of the kernel: q [B,Sq,Hq,D], k/v [B,Sk,Hkv,D] → (o [B,Sq,Hq,D], lse2 [B,Hq,Sq])."""
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    rep = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    s = torch.einsum("bhqd,bhkd->bhqk", qf, kf) * scale
    qi = torch.arange(Sq, device=q.device)[:, None]
    ki = torch.arange(Sk, device=q.device)[None, :]
    ok = torch.ones(Sq, Sk, dtype=torch.bool, device=q.device)
    if mask == "causal":
        ok = ki <= qi + causal_off
    elif mask == "block_causal":
        ok = (ki // frame) <= (qi // frame)
    if bias is not None:
        s = s + bias.float()
    s = s.masked_fill(~ok, float("-inf"))
    if key_valid is not None:
        s = s.masked_fill(~key_valid.bool()[:, None, None, :], float("-inf"))
    m = s.amax(-1, keepdim=True)
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    p = torch.exp(s - m)
    l = p.sum(-1, keepdim=True)
    o = torch.einsum("bhqk,bhkd->bhqd", p / l.clamp_min(1e-30), vf)
    lse2 = (m + torch.log(l)).squeeze(-1) * 1.4426950408889634
    return o.permute(0, 2, 1, 3).contiguous(), lse2


FWD_AUTO, FWD_ONE_TILE, FWD_TWO_TILE = 0, 1, 2


def set_forward_mode(mode: int) -> int:
    """Selects the forward kernel: by problem size (default), one 128-query tile per CTA, or two tiles per CTA
    ping-ponging on the tensor core (csrc/attention_fwd2_tcgen05.cu).  Returns the previous setting."""
    return int(cuda_lib().nb_flash_attn_fwd_mode(ctypes.c_int(mode)))


def set_backward_mode(mode: int) -> int:
    """Backward kernels: 0 = second generation (P / dS in tensor memory, transposed tiles for dK / dV), 1 = first
    generation.  Returns the previous setting."""
    return int(cuda_lib().nb_flash_attn_bwd_mode(ctypes.c_int(mode)))


def flash_attention_forward(q, k, v, scale=None, mask=None, frame=0, causal_off=0, key_valid=None, bias=None,
                            out=None, want_lse=True):
    """q [B,Sq,Hq,D], k/v [B,Sk,Hkv,D] bf16 (any batch/token/head strides, unit stride on D; views into a
    packed QKV buffer are fine).  Returns (o [B,Sq,Hq,D] bf16, lse2 [B,Hq,Sq] fp32 or None)."""
    assert q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    assert q.stride(3) == 1 and k.stride(3) == 1 and v.stride(3) == 1
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if out is None:
        out = torch.empty(B, Sq, Hq, D, device=q.device, dtype=torch.bfloat16)
    assert out.stride(3) == 1 and out.stride(2) == D and out.stride(0) == Sq * out.stride(1)
    lse = torch.empty(B, Hq, Sq, device=q.device, dtype=torch.float32) if want_lse else None
    kv = None
    if key_valid is not None:
        kv = key_valid.to(torch.uint8).contiguous()
        assert kv.shape == (B, Sk)
    if bias is not None:
        bias = bias.float().contiguous()
        assert bias.shape == (Sq, Sk)
    check(cuda_lib().nb_flash_attn_fwd(
        ptr(q), ptr(k), ptr(v), ptr(out), ptr(lse), ctypes.c_int(B), ctypes.c_int(Hq), ctypes.c_int(Hkv),
        ctypes.c_int(Sq), ctypes.c_int(Sk), ctypes.c_int(D),
        ctypes.c_longlong(q.stride(0)), ctypes.c_longlong(q.stride(1)), ctypes.c_longlong(q.stride(2)),
        ctypes.c_longlong(k.stride(0)), ctypes.c_longlong(k.stride(1)), ctypes.c_longlong(k.stride(2)),
        ctypes.c_longlong(v.stride(0)), ctypes.c_longlong(v.stride(1)), ctypes.c_longlong(v.stride(2)),
        ctypes.c_longlong(out.stride(1)), ctypes.c_float(scale), ctypes.c_int(MASK[mask]), ctypes.c_int(frame),
        ctypes.c_int(causal_off), ptr(kv), ptr(bias), ptr(device_status(q.device)), stream_ptr()), "flash_attn_fwd")
    return out, lse


def flash_attention_backward(q, k, v, o, lse, do, scale=None, mask=None, frame=0, causal_off=0, key_valid=None,
                             bias=None, dq=None, dk=None, dv=None):
    """Gradients of ``flash_attention_forward``: returns (dq, dk, dv) bf16 with the shapes of q, k, v."""
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if do.dtype != torch.bfloat16:
        do = do.to(torch.bfloat16)
    if do.stride(3) != 1:
        do = do.contiguous()
    assert o.stride(3) == 1 and o.stride(2) == D and o.stride(0) == Sq * o.stride(1)
    assert do.stride(0) == Sq * do.stride(1) or B == 1
    # outputs may be views into a packed dQKV buffer: head stride D, batch stride S * token pitch
    if dq is None:
        dq = torch.empty(B, Sq, Hq, D, device=q.device, dtype=torch.bfloat16)
    if dk is None:
        dk = torch.empty(B, Sk, Hkv, D, device=q.device, dtype=torch.bfloat16)
    if dv is None:
        dv = torch.empty(B, Sk, Hkv, D, device=q.device, dtype=torch.bfloat16)
    for t, S_ in ((dq, Sq), (dk, Sk), (dv, Sk)):
        assert t.stride(3) == 1 and t.stride(2) == D and (B == 1 or t.stride(0) == S_ * t.stride(1))
    delta = torch.empty(B, Hq, Sq, device=q.device, dtype=torch.float32)
    kv = key_valid.to(torch.uint8).contiguous() if key_valid is not None else None
    bs = bias.float().contiguous() if bias is not None else None
    L = ctypes.c_longlong
    check(cuda_lib().nb_flash_attn_bwd(
        ptr(q), ptr(k), ptr(v), ptr(o), ptr(do), ptr(lse), ptr(delta), ptr(dq), ptr(dk), ptr(dv),
        ctypes.c_int(B), ctypes.c_int(Hq), ctypes.c_int(Hkv), ctypes.c_int(Sq), ctypes.c_int(Sk), ctypes.c_int(D),
        L(q.stride(0)), L(q.stride(1)), L(q.stride(2)), L(k.stride(0)), L(k.stride(1)), L(k.stride(2)),
        L(v.stride(0)), L(v.stride(1)), L(v.stride(2)), L(o.stride(1)), L(do.stride(0)), L(do.stride(1)),
        L(do.stride(2)), L(dq.stride(1)), L(dk.stride(1)), L(dv.stride(1)), ctypes.c_float(scale),
        ctypes.c_int(MASK[mask]), ctypes.c_int(frame), ctypes.c_int(causal_off), ptr(kv), ptr(bs),
        ptr(device_status(q.device)), stream_ptr()), "flash_attn_bwd")
    return dq, dk, dv
