"""Transformer leaves: norms, embedding, RoPE, attention, feed-forward blocks.

CUDA path: norms.cu / misc_ops.cu / attention_tcgen05.cu / gemm_tcgen05.cu through ``noeira_b200.ops``.
CPU path: fp32 PyTorch (the oracle).  Parameter names follow the reference (``gamma``/``beta`` for norms,
``weight`` for embeddings — noeira/nn/primitives/layer_norm.mojo, rms_norm.mojo, embedding.mojo).
"""
from __future__ import annotations

import ctypes
import math

import torch

from .. import ops
from .._native import check, cuda_lib, ptr, stream_ptr
from ..ops.attention import attention_reference, flash_attention_backward, flash_attention_forward
from .init import Constant, Normal, Zero
from .layers import Linear
from .module import Module

_WS = {}


def _scratch(device, n):
    from ..ops.streams import ws_key
    key = ws_key(device)
    t = _WS.get(key)
    if t is None or t.numel() < n:
        t = torch.empty(max(n, 1 << 20), dtype=torch.float32, device=device)
        _WS[key] = t
    return t


class _Norm(Module):
    RMS = False

    def __init__(self, dim: int, eps: float = 1e-5, affine: bool = True):
        super().__init__()
        self.dim, self.eps, self.affine = dim, eps, affine
        self.gamma = self.add_param("gamma", (dim,), decay=False, init=Constant(1.0)) if affine else None
        self.beta = self.add_param("beta", (dim,), decay=False, init=Zero()) if (affine and not self.RMS) else None

    def forward(self, x):
        self._shape = x.shape
        x2 = x.reshape(-1, self.dim)
        if not self.on_cuda:
            xf = x2.float()
            if self.RMS:
                self._mean = torch.zeros(xf.shape[0], 1)
                self._rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
            else:
                self._mean = xf.mean(-1, keepdim=True)
                self._rstd = torch.rsqrt(xf.var(-1, unbiased=False, keepdim=True) + self.eps)
            self._xhat = (xf - self._mean) * self._rstd
            y = self._xhat * (self.gamma.data if self.gamma is not None else 1.0)
            if self.beta is not None:
                y = y + self.beta.data
            return y.reshape(self._shape)
        x2 = x2 if x2.stride(-1) == 1 else x2.contiguous()
        self._x = x2
        y = torch.empty(x2.shape[0], self.dim, device=x.device, dtype=torch.bfloat16)
        self._stats = torch.empty(x2.shape[0], 2, device=x.device, dtype=torch.float32)
        check(cuda_lib().nb_norm_fwd(ptr(x2), ctypes.c_int(x2.stride(0)), ptr(self.gamma.storage if self.gamma else None),
                                     ptr(self.beta.storage if self.beta else None), ptr(y), ctypes.c_int(self.dim),
                                     ptr(self._stats), ctypes.c_int(x2.shape[0]), ctypes.c_int(self.dim),
                                     ctypes.c_float(self.eps), ctypes.c_int(int(self.RMS)), stream_ptr()), "norm_fwd")
        return y.reshape(self._shape)

    def vjp(self, dy):
        dy2 = dy.reshape(-1, self.dim)
        if not self.on_cuda:
            g = dy2.float() * (self.gamma.data if self.gamma is not None else 1.0)
            if self.gamma is not None and not self.gamma.frozen:
                self.gamma.grad.add_((dy2.float() * self._xhat).sum(0))
            if self.beta is not None and not self.beta.frozen:
                self.beta.grad.add_(dy2.float().sum(0))
            m1 = torch.zeros_like(g[:, :1]) if self.RMS else g.mean(-1, keepdim=True)
            m2 = (g * self._xhat).mean(-1, keepdim=True)
            return (self._rstd * (g - m1 - self._xhat * m2)).reshape(self._shape)
        dy2 = dy2 if (dy2.stride(-1) == 1 and dy2.dtype == torch.bfloat16) else dy2.to(torch.bfloat16).contiguous()
        M = dy2.shape[0]
        dx = torch.empty(M, self.dim, device=dy.device, dtype=torch.bfloat16)
        lib = cuda_lib()
        split = lib.nb_norm_split(ctypes.c_int(M))
        want_g = self.gamma is not None and not self.gamma.frozen
        check(lib.nb_norm_bwd(ptr(self._x), ctypes.c_int(self._x.stride(0)), ptr(dy2), ctypes.c_int(dy2.stride(0)),
                              ptr(self.gamma.storage if self.gamma else None), ptr(self._stats), ptr(dx),
                              ctypes.c_int(self.dim), ptr(self.gamma.grad_storage if want_g else None),
                              ptr(self.beta.grad_storage if (self.beta is not None and want_g) else None),
                              ptr(_scratch(dy.device, 2 * split * self.dim)), ctypes.c_int(M), ctypes.c_int(self.dim),
                              ctypes.c_int(int(self.RMS)), ctypes.c_int(0), stream_ptr()), "norm_bwd")
        return dx.reshape(self._shape)

    def _release(self):
        self._x = self._stats = None


class LayerNorm(_Norm):
    RMS = False


class RMSNorm(_Norm):
    RMS = True


class Embedding(Module):
    def __init__(self, vocab: int, dim: int, scale: float = 1.0, std: float = 0.02):
        super().__init__()
        self.vocab, self.dim, self.scale = vocab, dim, scale
        self.weight = self.add_param("weight", (vocab, dim), decay=False, init=Normal(0.0, std))

    def forward(self, idx):
        self._idx = idx.reshape(-1).to(torch.int64)
        if not self.on_cuda:
            return (self.weight.data[self._idx] * self.scale).reshape(*idx.shape, self.dim)
        W = self.weight.shadow
        out = torch.empty(self._idx.numel(), self.dim, device=idx.device, dtype=torch.bfloat16)
        check(cuda_lib().nb_embedding_fwd(ptr(W), ctypes.c_int(W.stride(0)), ptr(self._idx), ptr(out), ctypes.c_int(self.dim),
                                          ctypes.c_int(self._idx.numel()), ctypes.c_int(self.dim), ctypes.c_float(self.scale),
                                          ctypes.c_int(self.weight.shape[0]), stream_ptr()), "embedding_fwd")
        return out.reshape(*idx.shape, self.dim)

    def vjp(self, dy):
        if self.weight.frozen:
            return None
        d2 = dy.reshape(-1, self.dim)
        if not self.on_cuda:
            self.weight.grad.index_add_(0, self._idx, d2.float() * self.scale)
            return None
        d2 = d2 if d2.stride(-1) == 1 else d2.contiguous()
        g = self.weight.grad_storage
        check(cuda_lib().nb_embedding_bwd(ptr(g), ctypes.c_int(g.stride(0)), ptr(self._idx), ptr(d2), ctypes.c_int(d2.stride(0)),
                                          ctypes.c_int(d2.shape[0]), ctypes.c_int(self.dim), ctypes.c_float(self.scale),
                                          ctypes.c_int(self.weight.shape[0]), stream_ptr()), "embedding_bwd")
        return None


def rope_(x, theta: float, pos0: int = 0, backward: bool = False):
    """In-place rotary embedding on a [B, S, H, D] view (rotate-half pairing)."""
    B, S, H, D = x.shape
    if x.is_cuda:
        assert x.stride(3) == 1
        check(cuda_lib().nb_rope(ptr(x), ctypes.c_int(B), ctypes.c_int(S), ctypes.c_int(H), ctypes.c_int(D),
                                 ctypes.c_longlong(x.stride(0)), ctypes.c_longlong(x.stride(1)),
                                 ctypes.c_longlong(x.stride(2)), ctypes.c_float(theta), ctypes.c_int(pos0),
                                 ctypes.c_int(int(backward)), stream_ptr()), "rope")
        return x
    half = D // 2
    inv = theta ** (-torch.arange(half, dtype=torch.float32) * 2.0 / D)
    ang = (pos0 + torch.arange(S, dtype=torch.float32))[:, None] * inv[None, :]
    sn, cs = ang.sin()[None, :, None, :], ang.cos()[None, :, None, :]
    if backward:
        sn = -sn
    x1, x2 = x[..., :half].clone(), x[..., half:].clone()
    x[..., :half] = x1 * cs - x2 * sn
    x[..., half:] = x2 * cs + x1 * sn
    return x


class AttentionCore:
    """softmax(scale·QKᵀ + mask)V with explicit backward (flash kernels on CUDA, fp32 reference on CPU)."""

    def __init__(self, mask=None, frame=0, causal_off=0, scale=None):
        self.mask, self.frame, self.causal_off, self.scale = mask, frame, causal_off, scale

    def forward(self, q, k, v, key_valid=None, bias=None):
        self._kv, self._bias = key_valid, bias
        if q.is_cuda:
            o, lse = flash_attention_forward(q, k, v, scale=self.scale, mask=self.mask, frame=self.frame,
                                             causal_off=self.causal_off, key_valid=key_valid, bias=bias)
            self._saved = (q, k, v, o, lse)
            return o
        self._leaf = tuple(t.detach().float().requires_grad_(True) for t in (q, k, v))
        with torch.enable_grad():
            o, _ = attention_reference(*self._leaf, scale=self.scale, mask=self.mask, frame=self.frame,
                                       causal_off=self.causal_off, key_valid=key_valid, bias=bias)
        self._out = o
        return o.detach()

    def vjp(self, do, dq=None, dk=None, dv=None):
        if do.is_cuda:
            q, k, v, o, lse = self._saved
            return flash_attention_backward(q, k, v, o, lse, do, scale=self.scale, mask=self.mask, frame=self.frame,
                                            causal_off=self.causal_off, key_valid=self._kv, bias=self._bias,
                                            dq=dq, dk=dk, dv=dv)
        return torch.autograd.grad(self._out, self._leaf, do.float())


class SelfAttention(Module):
    """Packed-QKV multi-head / grouped-query self-attention with optional RoPE.
    Children: ``qkv`` Linear(dim → (Hq + 2·Hkv)·hd), ``out`` Linear(Hq·hd → dim)."""

    def __init__(self, dim, heads, kv_heads=None, head_dim=None, mask=None, frame=0, rope_theta=None, bias=True):
        super().__init__()
        self.dim, self.h, self.hkv = dim, heads, kv_heads or heads
        self.hd = head_dim or dim // heads
        self.rope_theta = rope_theta
        self.qkv = self.add_child("qkv", Linear(dim, (self.h + 2 * self.hkv) * self.hd, bias=bias))
        self.out = self.add_child("out", Linear(self.h * self.hd, dim, bias=bias))
        self.core = AttentionCore(mask=mask, frame=frame)

    def forward(self, x, key_valid=None, bias=None, residual=None):
        B, S, _ = x.shape
        qkv = self.qkv.forward(x).reshape(B, S, self.h + 2 * self.hkv, self.hd)
        q, k, v = qkv[:, :, : self.h], qkv[:, :, self.h: self.h + self.hkv], qkv[:, :, self.h + self.hkv:]
        if self.rope_theta:
            rope_(q, self.rope_theta)
            rope_(k, self.rope_theta)
        self.last_k, self.last_v = k, v      # post-RoPE keys / values (prefix KV cache of a VLA)
        o = self.core.forward(q, k, v, key_valid=key_valid, bias=bias)
        return self.out.forward(o.reshape(B, S, self.h * self.hd), residual=residual)

    def vjp(self, dy):
        B, S, _ = dy.shape
        do = self.out.vjp(dy).reshape(B, S, self.h, self.hd)
        if dy.is_cuda:
            dqkv = torch.empty(B, S, self.h + 2 * self.hkv, self.hd, device=dy.device, dtype=torch.bfloat16)
            dq, dk, dv = dqkv[:, :, : self.h], dqkv[:, :, self.h: self.h + self.hkv], dqkv[:, :, self.h + self.hkv:]
            self.core.vjp(do, dq=dq, dk=dk, dv=dv)
        else:
            dq, dk, dv = self.core.vjp(do)
            dqkv = torch.cat([dq, dk, dv], dim=2)
            dq, dk = dqkv[:, :, : self.h], dqkv[:, :, self.h: self.h + self.hkv]
        if self.rope_theta:
            rope_(dq, self.rope_theta, backward=True)
            rope_(dk, self.rope_theta, backward=True)
        return self.qkv.vjp(dqkv.reshape(B, S, -1))


class CrossAttention(Module):
    """Q from ``x`` (+ optional positional term on q), K from ``mem_k`` and V from ``mem_v`` with separate
    projections q / k / v / out (the DETR wiring used by ACT: positions added to q and k but not to v,
    noeira/deep_agents/act/layers.mojo:86-107).  ``kv_dim`` lets the memory width differ (VLA expert)."""

    def __init__(self, dim, heads, kv_dim=None, kv_heads=None, head_dim=None, out_dim=None, bias=True):
        super().__init__()
        self.h, self.hkv = heads, kv_heads or heads
        self.hd = head_dim or dim // heads
        kv_dim = kv_dim or dim
        self.q = self.add_child("q", Linear(dim, self.h * self.hd, bias=bias))
        self.k = self.add_child("k", Linear(kv_dim, self.hkv * self.hd, bias=bias))
        self.v = self.add_child("v", Linear(kv_dim, self.hkv * self.hd, bias=bias))
        self.out = self.add_child("out", Linear(self.h * self.hd, out_dim or dim, bias=bias))
        self.core = AttentionCore()

    def forward(self, xq, mem_k, mem_v, key_valid=None):
        B, Sq, _ = xq.shape
        Sk = mem_k.shape[1]
        q = self.q.forward(xq).reshape(B, Sq, self.h, self.hd)
        k = self.k.forward(mem_k).reshape(B, Sk, self.hkv, self.hd)
        v = self.v.forward(mem_v).reshape(B, Sk, self.hkv, self.hd)
        o = self.core.forward(q, k, v, key_valid=key_valid)
        return self.out.forward(o.reshape(B, Sq, self.h * self.hd))

    def vjp(self, dy):
        """Returns (d xq, d mem_k, d mem_v)."""
        B, Sq, _ = dy.shape
        do = self.out.vjp(dy).reshape(B, Sq, self.h, self.hd)
        dq, dk, dv = self.core.vjp(do)
        Sk = dk.shape[1]
        return (self.q.vjp(dq.reshape(B, Sq, -1)), self.k.vjp(dk.reshape(B, Sk, -1)), self.v.vjp(dv.reshape(B, Sk, -1)))


class SwiGLU(Module):
    """h = silu(gate) ⊙ up for an input ``[.., 2H]`` laid out ``[gate | up]`` (noeira/nn/primitives/swiglu.mojo:42,63)."""

    def __init__(self, hidden):
        super().__init__()
        self.hidden = hidden

    def forward(self, gu):
        self._shape = gu.shape
        g2 = gu.reshape(-1, 2 * self.hidden)
        self._gu = g2
        if not gu.is_cuda:
            g, u = g2[:, : self.hidden].float(), g2[:, self.hidden:].float()
            return (torch.nn.functional.silu(g) * u).reshape(*self._shape[:-1], self.hidden)
        h = torch.empty(g2.shape[0], self.hidden, device=gu.device, dtype=torch.bfloat16)
        check(cuda_lib().nb_swiglu_fwd(ptr(g2), ctypes.c_int(g2.stride(0)), ptr(h), ctypes.c_int(self.hidden),
                                       ctypes.c_int(g2.shape[0]), ctypes.c_int(self.hidden), stream_ptr()), "swiglu_fwd")
        return h.reshape(*self._shape[:-1], self.hidden)

    def vjp(self, dh):
        d2 = dh.reshape(-1, self.hidden)
        if not dh.is_cuda:
            g, u = self._gu[:, : self.hidden].float(), self._gu[:, self.hidden:].float()
            sg = torch.sigmoid(g)
            dg = d2.float() * u * sg * (1 + g * (1 - sg))
            du = d2.float() * g * sg
            return torch.cat([dg, du], -1).reshape(self._shape)
        d2 = d2 if d2.stride(-1) == 1 else d2.contiguous()
        dgu = torch.empty_like(self._gu)
        check(cuda_lib().nb_swiglu_bwd(ptr(self._gu), ctypes.c_int(self._gu.stride(0)), ptr(d2), ctypes.c_int(d2.stride(0)),
                                       ptr(dgu), ctypes.c_int(d2.shape[0]), ctypes.c_int(self.hidden), stream_ptr()),
              "swiglu_bwd")
        return dgu.reshape(self._shape)


class SwiGLUFFN(Module):
    """Linear(D → 2H) → SwiGLU → Linear(H → D) (noeira/deep_agents/dreamer4/blocks.mojo:66-73)."""

    def __init__(self, dim, hidden, bias=False):
        super().__init__()
        self.up = self.add_child("0", Linear(dim, 2 * hidden, bias=bias))
        self.act = SwiGLU(hidden)
        self.down = self.add_child("1", Linear(hidden, dim, bias=bias))

    def forward(self, x, residual=None):
        return self.down.forward(self.act.forward(self.up.forward(x)), residual=residual)

    def vjp(self, dy):
        return self.up.vjp(self.act.vjp(self.down.vjp(dy)))


class FeedForward(Module):
    """Linear+activation (fused epilogue) → Linear; children ``0`` / ``1`` (FeedForwardGELU of the reference)."""

    def __init__(self, dim, hidden, act="gelu", bias=True):
        super().__init__()
        self.l0 = self.add_child("0", Linear(dim, hidden, act=act, bias=bias))
        self.l1 = self.add_child("1", Linear(hidden, dim, bias=bias))

    def forward(self, x, residual=None):
        return self.l1.forward(self.l0.forward(x), residual=residual)

    def vjp(self, dy):
        fuse = None
        if self.l0.on_cuda and self.l0._saved is not None and self.l0._saved.dtype == torch.bfloat16:
            fuse = (self.l0.act, self.l0._saved)
        return self.l0.vjp(self.l1.vjp(dy, fuse_dact=fuse), dy_is_pre=fuse is not None)


class TransformerBlock(Module):
    """Pre-norm block: x + Attn(norm(x)); x + FFN(norm(x)).  ``norm``: "layer" | "rms"; ``ffn``: "gelu" | "swiglu"."""

    def __init__(self, dim, heads, ff, kv_heads=None, head_dim=None, norm="layer", ffn="gelu", mask=None, frame=0,
                 rope_theta=None, bias=True, eps=1e-5):
        super().__init__()
        N = RMSNorm if norm == "rms" else LayerNorm
        self.n1 = self.add_child("norm1", N(dim, eps))
        self.attn = self.add_child("attn", SelfAttention(dim, heads, kv_heads, head_dim, mask, frame, rope_theta, bias))
        self.n2 = self.add_child("norm2", N(dim, eps))
        self.ffn = self.add_child("ffn", SwiGLUFFN(dim, ff, bias=bias) if ffn == "swiglu" else FeedForward(dim, ff, ffn, bias))

    def forward(self, x, key_valid=None, bias=None):
        x = self.attn.forward(self.n1.forward(x), key_valid=key_valid, bias=bias, residual=x)
        return self.ffn.forward(self.n2.forward(x), residual=x)

    def vjp(self, dy):
        d = dy + self.n2.vjp(self.ffn.vjp(dy))
        return d + self.n1.vjp(self.attn.vjp(d))


# ------------------------------------------------------------------------------------------ losses
class MSELoss:
    """mean over (rows × real columns) of (pred − target)²; writes dpred (bf16) and adds to a device accumulator."""

    def __init__(self, l1: bool = False):
        self.l1 = l1

    def __call__(self, pred, target, loss_acc, n_real=None, rowmask=None, weight=1.0):
        M, N = pred.reshape(-1, pred.shape[-1]).shape
        p2, t2 = pred.reshape(M, N), target.reshape(M, N).float()
        n_real = n_real or N
        denom = float(M * n_real)
        if not pred.is_cuda:
            d = (p2.float() - t2)[:, :n_real]
            if rowmask is not None:
                d = d * rowmask.reshape(M, 1)
            loss_acc += weight * (d.abs().sum() if self.l1 else (d * d).sum()) / denom
            g = torch.zeros(M, N)
            g[:, :n_real] = (d.sign() if self.l1 else 2 * d) * (weight / denom)
            return g.reshape(pred.shape)
        if p2.dtype not in (torch.bfloat16, torch.float32):
            p2 = p2.float()
        p2 = p2 if p2.stride(-1) == 1 else p2.contiguous()
        t2 = t2.contiguous()
        dp = torch.empty(M, N, device=pred.device, dtype=torch.bfloat16)
        check(cuda_lib().nb_mse_loss(ptr(p2), ctypes.c_int(p2.stride(0)), ptr(t2), ctypes.c_int(N), ptr(rowmask), ptr(dp),
                                     ctypes.c_int(N), ptr(_scratch(pred.device, 2048)), ptr(loss_acc), ctypes.c_int(M),
                                     ctypes.c_int(N), ctypes.c_int(n_real), ctypes.c_float(weight / denom),
                                     ctypes.c_float(weight / denom), ctypes.c_int(int(self.l1)),
                                     ctypes.c_int(int(p2.dtype == torch.float32)), stream_ptr()), "mse_loss")
        return dp.reshape(pred.shape)


def cross_entropy(logits, target, loss_acc, ignore_index=-100):
    """Mean softmax cross-entropy; on CUDA the gradient OVERWRITES ``logits`` (bf16) and is returned."""
    M, V = logits.reshape(-1, logits.shape[-1]).shape
    tg = target.reshape(-1).to(torch.int64)
    n = max(int((tg != ignore_index).sum().item()) if not logits.is_cuda else M, 1)
    if not logits.is_cuda:
        lf = logits.reshape(M, V).float().detach().requires_grad_(True)
        with torch.enable_grad():
            loss = torch.nn.functional.cross_entropy(lf, tg, ignore_index=ignore_index, reduction="sum") / n
        loss_acc += loss.detach()
        return torch.autograd.grad(loss, lf)[0].reshape(logits.shape)
    l2 = logits.reshape(M, V)
    assert l2.stride(-1) == 1
    check(cuda_lib().nb_cross_entropy(ptr(l2), ctypes.c_int(l2.stride(0)), ptr(tg), ctypes.c_int(M), ctypes.c_int(V),
                                      ptr(_scratch(logits.device, M)), ptr(loss_acc), ctypes.c_float(1.0 / n),
                                      ctypes.c_float(1.0 / n), ctypes.c_longlong(ignore_index), ctypes.c_int(1),
                                      stream_ptr()), "cross_entropy")
    return logits


def sincos_embed(t, dim, min_period=4e-3, max_period=4.0):
    """[B] → [B, dim] sinusoidal embedding with geometric periods (noeira/deep_agents/smolvla/embed.mojo:55-56)."""
    B = t.numel()
    if t.is_cuda:
        out = torch.empty(B, dim, device=t.device, dtype=torch.bfloat16)
        check(cuda_lib().nb_sincos_embed(ptr(t.float().contiguous()), ptr(out), ctypes.c_int(dim), ctypes.c_int(B),
                                         ctypes.c_int(dim), ctypes.c_float(min_period), ctypes.c_float(max_period),
                                         stream_ptr()), "sincos_embed")
        return out
    half = dim // 2
    frac = torch.linspace(0, 1, half) if half > 1 else torch.zeros(1)
    period = min_period * (max_period / min_period) ** frac
    a = t.float()[:, None] * 2 * math.pi / period[None, :]
    return torch.cat([a.sin(), a.cos()], -1)
