"""Convolutional leaves on the NHWC bf16 path: Conv2D (patch gather + tcgen05 GEMM with fused bias / ReLU),
BatchNorm2D (training statistics, fused ReLU and residual add), MaxPool2D, and the torchvision-topology
ResNet-18 backbone used by ACT (noeira/nn/models/resnet18.mojo:142: stride 32, trainable BatchNorm).

Activations are ``[B, H, W, C]``.  ``Conv2D.weight`` is kept in GEMM layout ``[KH·KW·IC, OC]`` in memory; files
hold the reference layout ``[OC, IC, KH, KW]`` (the parameter carries export / import hooks that permute).
"""
from __future__ import annotations

import ctypes
import os

import torch

from .. import ops
from .._native import check, cuda_lib, ptr, stream_ptr
from .init import Constant, Kaiming, Zero
from .layers import colsum_into
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


class Conv2D(Module):
    def __init__(self, ic, oc, k, stride=1, pad=0, bias=True, relu=False, need_input_grad=True):
        super().__init__()
        self.ic, self.oc, self.k, self.stride, self.pad, self.relu = ic, oc, k, stride, pad, relu
        self.icp = (ic + 7) // 8 * 8          # channels as stored (stem: 3 → 8, extra channels are zero)
        self.need_input_grad = need_input_grad
        self.force_implicit = False
        self.implicit_gemm = os.environ.get("NOEIRA_B200_IMPLICIT_CONV", "1") != "0"
        # weight gradient straight from the NHWC input (no patch matrix in the backward either)
        self.implicit_wgrad = os.environ.get("NOEIRA_B200_IMPLICIT_WGRAD", "0") == "1"
        self.weight = self.add_param("weight", (k * k * self.icp, oc), decay=True, init=Kaiming(), fan_in=ic * k * k,
                                     fan_out=oc)
        if self.icp != ic:
            w = self.weight.data.view(k * k, self.icp, oc)
            w[:, ic:, :] = 0
        self.bias = self.add_param("bias", (oc,), decay=False, init=Zero()) if bias else None
        icp, KK = self.icp, k
        self.weight.to_file = lambda t: t.view(KK, KK, icp, oc)[:, :, :ic, :].permute(3, 2, 0, 1).contiguous()
        self.weight.from_file = lambda t: torch.nn.functional.pad(t.reshape(oc, ic, KK, KK).permute(2, 3, 1, 0),
                                                                  (0, 0, 0, icp - ic)).reshape(KK * KK * icp, oc)

    def _implicit_ok(self, C, OW):
        if self.stride != 1 or C % 64 or not self.implicit_gemm:
            return False
        # a trainable layer needs the patch matrix for its weight gradient anyway; building it in the forward and
        # reusing it measured 0.3 ms faster per ACT step than implicit forward + rebuild in the backward
        if self.training and torch.is_grad_enabled() and not self.weight.frozen and not self.force_implicit \
                and not (self.implicit_wgrad and self._implicit_wgrad_ok(OW)):
            return False
        bw = 1
        while bw < 128 and OW % (bw * 2) == 0:
            bw *= 2
        return bw >= 16          # runs of 8 pixels need 16 TMA boxes per stage and measured slower than the patch matrix

    def _patches(self):
        """Patch matrix [B·OH·OW, KH·KW·C] of the saved input (backward of the implicit-GEMM forward)."""
        x = self._xin
        B, H, W, C = x.shape
        OH, OW = self.out_hw(H, W)
        K = self.k * self.k * C
        if self.k == 1 and self.pad == 0:
            return x.reshape(B * OH * OW, C)
        col = torch.empty(B * OH * OW, K, device=x.device, dtype=torch.bfloat16)
        check(cuda_lib().nb_im2col(ptr(x), ptr(col), *(ctypes.c_int(v) for v in (B, H, W, C, self.k, self.k, self.stride,
                                                                               self.pad, OH, OW, K)), stream_ptr()), "im2col")
        return col

    def out_hw(self, H, W):
        return (H + 2 * self.pad - self.k) // self.stride + 1, (W + 2 * self.pad - self.k) // self.stride + 1

    def forward(self, x):
        B, H, W, C = x.shape
        assert C == self.icp, (C, self.icp)
        OH, OW = self.out_hw(H, W)
        self._in = (B, H, W)
        if not self.on_cuda:
            self._x = x.float()
            w = self.weight.data.view(self.k, self.k, self.icp, self.oc).permute(3, 2, 0, 1)
            y = torch.nn.functional.conv2d(self._x.permute(0, 3, 1, 2), w, self.bias.data if self.bias is not None else None,
                                           self.stride, self.pad).permute(0, 2, 3, 1)
            self._y = torch.relu(y) if self.relu else y
            return self._y
        M, K = B * OH * OW, self.k * self.k * C
        if self._implicit_ok(C, OW):
            # implicit GEMM: the GEMM's TMA producer reads the patches straight from x (no patch matrix in memory);
            # the backward pass rebuilds the patch matrix only if a weight gradient is needed
            xc = x if x.is_contiguous() else x.contiguous()
            y = torch.empty(M, self.weight.shadow.shape[1], device=x.device, dtype=torch.bfloat16)
            from ..ops.status import device_status
            from ..ops.gemm import ACT
            check(cuda_lib().nb_conv_implicit_fwd(ptr(xc), ptr(self.weight.shadow), ptr(y), *(ctypes.c_int(v) for v in (
                B, H, W, C, self.oc, self.k, self.k, self.pad, self.weight.shadow.stride(0), y.stride(0))),
                ptr(self.bias.storage if self.bias is not None else None), ctypes.c_int(ACT["relu" if self.relu else None]),
                None, ctypes.c_int(0), ptr(device_status(x.device)), stream_ptr()), "conv_implicit_fwd")
            self._col, self._xin, self._y = None, xc, y
            return y[:, : self.oc].reshape(B, OH, OW, self.oc) if y.shape[1] != self.oc else y.view(B, OH, OW, self.oc)
        self._xin = None
        if self.k == 1 and self.stride == 1 and self.pad == 0:
            col = x.reshape(M, C)
        else:
            col = torch.empty(M, K, device=x.device, dtype=torch.bfloat16)
            xc = x if x.is_contiguous() else x.contiguous()
            check(cuda_lib().nb_im2col(ptr(xc), ptr(col), *(ctypes.c_int(v) for v in (B, H, W, C, self.k, self.k, self.stride,
                                                                                   self.pad, OH, OW, K)), stream_ptr()), "im2col")
        self._col = col
        y = ops.gemm(col, self.weight.shadow, b_mn=True, bias=self.bias.storage if self.bias is not None else None,
                     act="relu" if self.relu else None)
        self._y = y
        return y[:, : self.oc].reshape(B, OH, OW, self.oc) if y.shape[1] != self.oc else y.view(B, OH, OW, self.oc)

    def vjp(self, dy):
        B, H, W = self._in
        OH, OW = self.out_hw(H, W)
        if not self.on_cuda:
            g = dy.float()
            if self.relu:
                g = g * (self._y > 0)
            w = self.weight.data.view(self.k, self.k, self.icp, self.oc).permute(3, 2, 0, 1)
            xn, gn = self._x.permute(0, 3, 1, 2), g.permute(0, 3, 1, 2)
            if not self.weight.frozen:
                gw = torch.nn.grad.conv2d_weight(xn, w.shape, gn, self.stride, self.pad)
                self.weight.grad.add_(gw.permute(2, 3, 1, 0).reshape(self.weight.shape))
                if self.bias is not None:
                    self.bias.grad.add_(g.sum((0, 1, 2)))
            if not self.need_input_grad:
                return None
            return torch.nn.grad.conv2d_input(xn.shape, w, gn, self.stride, self.pad).permute(0, 2, 3, 1)
        M = B * OH * OW
        d2 = dy.reshape(M, self.oc)
        d2 = d2 if (d2.stride(-1) == 1 and d2.dtype == torch.bfloat16) else d2.to(torch.bfloat16).contiguous()
        if self.relu:
            from .layers import act_backward
            d2 = act_backward(d2.contiguous(), self._y[:, : self.oc].contiguous() if self._y.shape[1] != self.oc else self._y, "relu")
        if not self.weight.frozen:
            if self._col is None and self._xin is not None and self.implicit_wgrad and self._implicit_wgrad_ok(OW):
                self._implicit_wgrad(d2, B, H, W)
            else:
                col = self._col if self._col is not None else self._patches()
                ops.gemm(col, d2, a_mn=True, b_mn=True, out=self.weight.grad_storage, accumulate=True, n=self.oc)
            if self.bias is not None:
                colsum_into(d2, self.bias.grad_storage, self.oc)
        if not self.need_input_grad:
            return None
        if self._implicit_dgrad_ok(W):
            return self._implicit_dgrad(d2, B, H, W, OH, OW)
        K = self.k * self.k * self.icp
        dcol = ops.gemm(d2, self.weight.shadow[:, : self.oc])           # [M, K]
        if self.k == 1 and self.stride == 1 and self.pad == 0:
            return dcol.view(B, H, W, self.icp)
        dx = torch.empty(B, H, W, self.icp, device=dy.device, dtype=torch.bfloat16)
        check(cuda_lib().nb_col2im(ptr(dcol), ptr(dx), *(ctypes.c_int(v) for v in (B, H, W, self.icp, self.k, self.k, self.stride,
                                                                               self.pad, OH, OW, K)), stream_ptr()), "col2im")
        return dx

    def _implicit_wgrad_ok(self, OW):
        bw = 1
        while bw < 64 and OW % (bw * 2) == 0:
            bw *= 2
        return self.stride == 1 and self.icp % 64 == 0 and bw >= 8

    def _implicit_wgrad(self, d2, B, H, W):
        """dW += patches(x)ᵀ · dy with the patches read by the GEMM's TMA producer from the saved NHWC input."""
        from ..ops.gemm import default_workspace
        from ..ops.status import device_status
        x, g = self._xin, self.weight.grad_storage
        d2 = d2 if (d2.stride(0) * 2) % 16 == 0 and d2.data_ptr() % 16 == 0 else d2.contiguous()
        ws = default_workspace(x.device)
        check(cuda_lib().nb_conv_implicit_wgrad(ptr(x), ptr(d2), ptr(g), *(ctypes.c_int(v) for v in (
            B, H, W, self.icp, self.oc, self.k, self.k, self.pad, d2.stride(0), g.stride(0))), ptr(device_status(x.device)),
            ptr(ws), ctypes.c_longlong(ws.numel()), stream_ptr()), "conv_implicit_wgrad")

    def _implicit_dgrad_ok(self, W):
        """Stride-1 layers with at least 64 output channels: the input gradient is itself a stride-1 convolution of
        dy (taps mirrored, channel roles swapped), which the implicit-GEMM kernel computes without the 9x larger
        patch-gradient matrix and the col2im pass over it."""
        if self.stride != 1 or self.k == 1 or self.oc % 64 or not self.implicit_gemm or 2 * self.pad > self.k - 1 + self.k - 1:
            return False
        bw = 1
        while bw < 128 and W % (bw * 2) == 0:
            bw *= 2
        return bw >= 8

    def _implicit_dgrad(self, d2, B, H, W, OH, OW):
        k, oc, icp = self.k, self.oc, self.icp
        # W'[(kh', kw', oc), ic] = W[(k-1-kh', k-1-kw', ic), oc]
        wt = self.weight.shadow[:, :oc].reshape(k, k, icp, oc).flip(0, 1).permute(0, 1, 3, 2).contiguous().view(k * k * oc, icp)
        dyc = d2 if d2.is_contiguous() else d2.contiguous()
        dx = torch.empty(B * H * W, icp, device=d2.device, dtype=torch.bfloat16)
        from ..ops.status import device_status
        check(cuda_lib().nb_conv_implicit_fwd(ptr(dyc), ptr(wt), ptr(dx), *(ctypes.c_int(v) for v in (
            B, OH, OW, oc, icp, k, k, k - 1 - self.pad, wt.stride(0), dx.stride(0))), None, ctypes.c_int(0), None,
            ctypes.c_int(0), ptr(device_status(d2.device)), stream_ptr()), "conv_implicit_dgrad")
        return dx.view(B, H, W, icp)

    def _release(self):
        self._col = self._y = self._xin = None


class BatchNorm2D(Module):
    """Per-channel batch statistics over (B, H, W) in training, running statistics in eval; optional fused ReLU and
    residual add: y = relu(bn(x) + residual).  Params ``gamma`` / ``beta``, states ``running_mean`` / ``running_var``."""

    def __init__(self, c, eps=1e-5, momentum=0.1, relu=False):
        super().__init__()
        self.c, self.eps, self.momentum, self.relu = c, eps, momentum, relu
        self.gamma = self.add_param("gamma", (c,), decay=False, init=Constant(1.0))
        self.beta = self.add_param("beta", (c,), decay=False, init=Zero())
        self.running_mean = self.add_state("running_mean", (c,), 0.0)
        self.running_var = self.add_state("running_var", (c,), 1.0)

    def forward(self, x, residual=None):
        shape = x.shape
        M = x.numel() // self.c
        self._has_res = residual is not None
        if not self.on_cuda:
            xf = x.float().reshape(M, self.c)
            if self.training:
                mean, var = xf.mean(0), xf.var(0, unbiased=False)
                self.running_mean.data.mul_(1 - self.momentum).add_(self.momentum * mean)
                self.running_var.data.mul_(1 - self.momentum).add_(self.momentum * var * M / max(M - 1, 1))
            else:
                mean, var = self.running_mean.data, self.running_var.data
            self._rstd = torch.rsqrt(var + self.eps)
            self._xhat = (xf - mean) * self._rstd
            y = self._xhat * self.gamma.data + self.beta.data
            if residual is not None:
                y = y + residual.float().reshape(M, self.c)
            self._y = torch.relu(y) if self.relu else y
            return self._y.reshape(shape)
        xc = x if x.is_contiguous() else x.contiguous()
        self._x = xc
        y = torch.empty_like(xc)
        self._mean = torch.empty(self.c, device=x.device) if self.training else self.running_mean.data
        self._rstdv = torch.empty(self.c, device=x.device) if self.training else torch.rsqrt(self.running_var.data + self.eps)
        lib = cuda_lib()
        split = lib.nb_bn_split(ctypes.c_longlong(M))
        rc = residual.contiguous() if residual is not None else None
        check(lib.nb_bn_fwd(ptr(xc), ptr(self.gamma.storage), ptr(self.beta.storage), ptr(rc), ptr(y), ptr(self._mean),
                            ptr(self._rstdv), ptr(self.running_mean.data), ptr(self.running_var.data),
                            ptr(_scratch(x.device, 2 * split * self.c)), ctypes.c_longlong(M), ctypes.c_int(self.c),
                            ctypes.c_float(self.eps), ctypes.c_float(self.momentum), ctypes.c_int(int(self.relu)),
                            ctypes.c_int(int(self.training)), stream_ptr()), "bn_fwd")
        self._y = y
        return y

    def vjp(self, dy):
        """Returns dx, or (dx, dresidual) when a residual was added in forward."""
        shape = dy.shape
        M = dy.numel() // self.c
        if not self.on_cuda:
            g = dy.float().reshape(M, self.c)
            if self.relu:
                g = g * (self._y > 0)
            self.gamma.grad.add_((g * self._xhat).sum(0))
            self.beta.grad.add_(g.sum(0))
            gg = g * self.gamma.data
            dx = self._rstd * (gg - gg.mean(0) - self._xhat * (gg * self._xhat).mean(0))
            dx = dx.reshape(shape)
            return (dx, g.reshape(shape)) if self._has_res else dx
        d = dy if (dy.is_contiguous() and dy.dtype == torch.bfloat16) else dy.to(torch.bfloat16).contiguous()
        dx = torch.empty_like(d)
        dres = torch.empty_like(d) if self._has_res else None
        lib = cuda_lib()
        split = lib.nb_bn_split(ctypes.c_longlong(M))
        ws = _scratch(dy.device, 2 * split * self.c + 2 * self.c)
        sums = ws[2 * split * self.c:]
        check(lib.nb_bn_bwd(ptr(d), ptr(self._x), ptr(self._y if self.relu else None), ptr(self._mean), ptr(self._rstdv),
                            ptr(self.gamma.storage), ptr(dx), ptr(dres), ptr(self.gamma.grad_storage), ptr(self.beta.grad_storage),
                            ptr(ws), ptr(sums), ctypes.c_longlong(M), ctypes.c_int(self.c), stream_ptr()), "bn_bwd")
        return (dx, dres) if self._has_res else dx


class MaxPool2D(Module):
    def __init__(self, k=3, stride=2, pad=1):
        super().__init__()
        self.k, self.stride, self.pad = k, stride, pad

    def forward(self, x):
        B, H, W, C = x.shape
        OH, OW = (H + 2 * self.pad - self.k) // self.stride + 1, (W + 2 * self.pad - self.k) // self.stride + 1
        self._dims = (B, H, W, C, OH, OW)
        if not x.is_cuda:
            y, idx = torch.nn.functional.max_pool2d(x.float().permute(0, 3, 1, 2), self.k, self.stride, self.pad, return_indices=True)
            self._idx = idx
            return y.permute(0, 2, 3, 1)
        xc = x if x.is_contiguous() else x.contiguous()
        y = torch.empty(B, OH, OW, C, device=x.device, dtype=torch.bfloat16)
        self._idx = torch.empty(B, OH, OW, C, device=x.device, dtype=torch.int32)
        check(cuda_lib().nb_maxpool_fwd(ptr(xc), ptr(y), ptr(self._idx), *(ctypes.c_int(v) for v in (B, H, W, C, self.k, self.stride,
                                                                                                 self.pad, OH, OW)), stream_ptr()), "maxpool_fwd")
        return y

    def vjp(self, dy):
        B, H, W, C, OH, OW = self._dims
        if not dy.is_cuda:
            # windows overlap (3x3 / stride 2): an input that is the maximum of several windows sums their gradients
            g = torch.zeros(B, C, H * W).scatter_add_(2, self._idx.reshape(B, C, -1),
                                                      dy.float().permute(0, 3, 1, 2).reshape(B, C, -1))
            return g.view(B, C, H, W).permute(0, 2, 3, 1)
        d = dy if (dy.is_contiguous() and dy.dtype == torch.bfloat16) else dy.to(torch.bfloat16).contiguous()
        dx = torch.empty(B, H, W, C, device=dy.device, dtype=torch.bfloat16)
        check(cuda_lib().nb_maxpool_bwd(ptr(d), ptr(self._idx), ptr(dx), *(ctypes.c_int(v) for v in (B, H, W, C, self.k, self.stride,
                                                                                                 self.pad, OH, OW)), stream_ptr()), "maxpool_bwd")
        return dx


class AvgPool2D(Module):
    """Non-overlapping K x K average pooling on NHWC (a trailing partial window is dropped)."""

    def __init__(self, k=2):
        super().__init__()
        self.k = k

    def forward(self, x):
        B, H, W, C = x.shape
        OH, OW = H // self.k, W // self.k
        self._in = (B, H, W, C)
        if not x.is_cuda:
            return x[:, : OH * self.k, : OW * self.k].reshape(B, OH, self.k, OW, self.k, C).float().mean((2, 4))
        xc = x if x.is_contiguous() else x.contiguous()
        y = torch.empty(B, OH, OW, C, device=x.device, dtype=torch.bfloat16)
        check(cuda_lib().nb_avgpool(ptr(xc), ptr(y), *(ctypes.c_int(v) for v in (B, H, W, C, self.k, OH, OW, 0)), stream_ptr()), "avgpool")
        return y

    def vjp(self, dy):
        B, H, W, C = self._in
        OH, OW = H // self.k, W // self.k
        if not dy.is_cuda:
            dx = torch.zeros(B, H, W, C)
            dx[:, : OH * self.k, : OW * self.k] = (dy.float() / (self.k * self.k)).repeat_interleave(self.k, 1).repeat_interleave(self.k, 2)
            return dx
        d = dy if (dy.is_contiguous() and dy.dtype == torch.bfloat16) else dy.to(torch.bfloat16).contiguous()
        dx = torch.empty(B, H, W, C, device=dy.device, dtype=torch.bfloat16)
        check(cuda_lib().nb_avgpool(ptr(d), ptr(dx), *(ctypes.c_int(v) for v in (B, H, W, C, self.k, OH, OW, 1)), stream_ptr()), "avgpool_bwd")
        return dx


class Upsample2D(Module):
    """Nearest-neighbour upsampling by an integer factor on NHWC."""

    def __init__(self, scale=2):
        super().__init__()
        self.s = scale

    def forward(self, x):
        B, H, W, C = x.shape
        self._in = (B, H, W, C)
        if not x.is_cuda:
            return x.repeat_interleave(self.s, 1).repeat_interleave(self.s, 2)
        xc = x if x.is_contiguous() else x.contiguous()
        y = torch.empty(B, H * self.s, W * self.s, C, device=x.device, dtype=torch.bfloat16)
        check(cuda_lib().nb_upsample_nearest(ptr(xc), ptr(y), *(ctypes.c_int(v) for v in (B, H, W, C, self.s, 0)), stream_ptr()), "upsample")
        return y

    def vjp(self, dy):
        B, H, W, C = self._in
        if not dy.is_cuda:
            return dy.float().reshape(B, H, self.s, W, self.s, C).sum((2, 4))
        d = dy if (dy.is_contiguous() and dy.dtype == torch.bfloat16) else dy.to(torch.bfloat16).contiguous()
        dx = torch.empty(B, H, W, C, device=dy.device, dtype=torch.bfloat16)
        check(cuda_lib().nb_upsample_nearest(ptr(d), ptr(dx), *(ctypes.c_int(v) for v in (B, H, W, C, self.s, 1)), stream_ptr()), "upsample_bwd")
        return dx


class Conv2DTranspose(Module):
    """Transposed convolution on NHWC: the adjoint of ``Conv2D(oc → ic, k, stride, pad)``.  Output size
    ``(H − 1)·stride − 2·pad + k``.  On CUDA the forward is the data-gradient path of the convolution (GEMM with the weight,
    then the deterministic gather-style col2im), the input gradient is the convolution's forward (patch gather + GEMM),
    the weight gradient one GEMM on the patches of dy.  Weight in the GEMM layout of the adjoint convolution
    ``[k·k·oc_pad, ic]``; files hold the torch layout ``[ic, oc, k, k]``.
    (noeira/nn/primitives/conv2d_transpose.mojo)"""

    def __init__(self, ic, oc, k, stride=1, pad=0, bias=True, relu=False, need_input_grad=True):
        super().__init__()
        self.ic, self.oc, self.k, self.stride, self.pad, self.relu = ic, oc, k, stride, pad, relu
        self.ocp = (oc + 7) // 8 * 8
        self.need_input_grad = need_input_grad
        self.weight = self.add_param("weight", (k * k * self.ocp, ic), decay=True, init=Kaiming(), fan_in=ic * k * k, fan_out=oc)
        if self.ocp != oc:
            self.weight.data.view(k * k, self.ocp, ic)[:, oc:, :] = 0
        self.bias = self.add_param("bias", (oc,), decay=False, init=Zero()) if bias else None
        ocp, KK = self.ocp, k
        self.weight.to_file = lambda t: t.view(KK, KK, ocp, ic)[:, :, :oc, :].permute(3, 2, 0, 1).contiguous()
        self.weight.from_file = lambda t: torch.nn.functional.pad(t.reshape(ic, oc, KK, KK).permute(2, 3, 1, 0),
                                                                  (0, 0, 0, ocp - oc)).reshape(KK * KK * ocp, ic)

    def out_hw(self, H, W):
        return (H - 1) * self.stride - 2 * self.pad + self.k, (W - 1) * self.stride - 2 * self.pad + self.k

    def _w_torch(self):
        return self.weight.data.view(self.k, self.k, self.ocp, self.ic)[:, :, : self.oc].permute(3, 2, 0, 1)      # [ic, oc, k, k]

    def forward(self, x):
        B, H, W, C = x.shape
        assert C == self.ic
        OH, OW = self.out_hw(H, W)
        self._in = (B, H, W)
        if not self.on_cuda:
            self._x = x.float()
            y = torch.nn.functional.conv_transpose2d(self._x.permute(0, 3, 1, 2), self._w_torch(),
                                                     self.bias.data if self.bias is not None else None, self.stride, self.pad).permute(0, 2, 3, 1)
            self._y = torch.relu(y) if self.relu else y
            return self._y
        M, K = B * H * W, self.k * self.k * self.ocp
        x2 = x.reshape(M, C)
        x2 = x2 if (x2.stride(-1) == 1 and x2.dtype == torch.bfloat16 and (x2.stride(0) * 2) % 16 == 0) else _rows16(x2)
        self._x2 = x2
        dcol = ops.gemm(x2, self.weight.shadow[:, : self.ic])                    # [M, K] = x · Wᵀ
        y = torch.empty(B, OH, OW, self.ocp, device=x.device, dtype=torch.bfloat16)
        check(cuda_lib().nb_col2im(ptr(dcol), ptr(y), *(ctypes.c_int(v) for v in (B, OH, OW, self.ocp, self.k, self.k, self.stride,
                                                                              self.pad, H, W, K)), stream_ptr()), "col2im")
        y = y[..., : self.oc]
        if self.bias is not None:
            y = y + self.bias.data.to(torch.bfloat16)
        if self.relu:
            y = torch.relu(y)
        self._y = y
        return y

    def vjp(self, dy):
        B, H, W = self._in
        OH, OW = self.out_hw(H, W)
        if not self.on_cuda:
            g = dy.float()
            if self.relu:
                g = g * (self._y > 0)
            gn, xn, w = g.permute(0, 3, 1, 2), self._x.permute(0, 3, 1, 2), self._w_torch()
            if not self.weight.frozen:
                gw = torch.nn.grad.conv2d_weight(gn, w.shape, xn, self.stride, self.pad)          # adjoint conv: input dy, output x
                self.weight.grad.view(self.k, self.k, self.ocp, self.ic)[:, :, : self.oc].add_(gw.permute(2, 3, 1, 0))
                if self.bias is not None:
                    self.bias.grad.add_(g.sum((0, 1, 2)))
            if not self.need_input_grad:
                return None
            return torch.nn.functional.conv2d(gn, w, None, self.stride, self.pad).permute(0, 2, 3, 1)
        g = dy
        if self.relu:
            g = g * (self._y > 0)
        M, K = B * H * W, self.k * self.k * self.ocp
        gp = torch.zeros(B, OH, OW, self.ocp, device=dy.device, dtype=torch.bfloat16)
        gp[..., : self.oc] = g
        col = torch.empty(M, K, device=dy.device, dtype=torch.bfloat16)
        check(cuda_lib().nb_im2col(ptr(gp), ptr(col), *(ctypes.c_int(v) for v in (B, OH, OW, self.ocp, self.k, self.k, self.stride,
                                                                              self.pad, H, W, K)), stream_ptr()), "im2col")
        if not self.weight.frozen:
            ops.gemm(col, self._x2, a_mn=True, b_mn=True, out=self.weight.grad_storage, accumulate=True, n=self.ic)
            if self.bias is not None:
                self.bias.grad_storage[: self.oc].add_(g.float().sum((0, 1, 2)))
        if not self.need_input_grad:
            return None
        dx = ops.gemm(col, self.weight.shadow, b_mn=True)
        return dx[:, : self.ic].reshape(B, H, W, self.ic)

    def _release(self):
        self._x = self._x2 = self._y = None


def _rows16(t):
    out = torch.zeros(t.shape[0], (t.shape[1] + 7) // 8 * 8, device=t.device, dtype=torch.bfloat16)
    out[:, : t.shape[1]] = t
    return out[:, : t.shape[1]]


class BasicBlock(Module):
    """conv3x3-bn-relu, conv3x3-bn, (+ 1x1 downsample), add, relu — children named as in torchvision."""

    def __init__(self, ic, oc, stride):
        super().__init__()
        self.conv1 = self.add_child("conv1", Conv2D(ic, oc, 3, stride, 1, bias=False))
        self.bn1 = self.add_child("bn1", BatchNorm2D(oc, relu=True))
        self.conv2 = self.add_child("conv2", Conv2D(oc, oc, 3, 1, 1, bias=False))
        self.bn2 = self.add_child("bn2", BatchNorm2D(oc, relu=True))
        self.down = None
        if stride != 1 or ic != oc:
            self.down = self.add_child("downsample.0", Conv2D(ic, oc, 1, stride, 0, bias=False))
            self.down_bn = self.add_child("downsample.1", BatchNorm2D(oc))

    def forward(self, x):
        idt = self.down_bn.forward(self.down.forward(x)) if self.down is not None else x
        h = self.bn1.forward(self.conv1.forward(x))
        return self.bn2.forward(self.conv2.forward(h), residual=idt)

    def vjp(self, dy):
        dh, dres = self.bn2.vjp(dy)
        dx = self.conv1.vjp(self.bn1.vjp(self.conv2.vjp(dh)))
        if self.down is not None:
            dx = dx + self.down.vjp(self.down_bn.vjp(dres))
        else:
            dx = dx + dres
        return dx


class ResNet18Backbone(Module):
    """Stem (7x7/2, bn, relu, maxpool 3x3/2) + 4 stages of 2 BasicBlocks (64, 128, 256, 512); output stride 32."""

    def __init__(self):
        super().__init__()
        self.conv1 = self.add_child("conv1", Conv2D(3, 64, 7, 2, 3, bias=False, need_input_grad=False))
        self.bn1 = self.add_child("bn1", BatchNorm2D(64, relu=True))
        self.pool = MaxPool2D(3, 2, 1)
        self.blocks = []
        ic = 64
        for li, (oc, stride) in enumerate(((64, 1), (128, 2), (256, 2), (512, 2)), start=1):
            for bi in range(2):
                blk = self.add_child(f"layer{li}.{bi}", BasicBlock(ic, oc, stride if bi == 0 else 1))
                self.blocks.append(blk)
                ic = oc

    def forward(self, x):
        h = self.pool.forward(self.bn1.forward(self.conv1.forward(x)))
        for b in self.blocks:
            h = b.forward(h)
        return h

    def vjp(self, dy):
        for b in reversed(self.blocks):
            dy = b.vjp(dy)
        self.conv1.vjp(self.bn1.vjp(self.pool.vjp(dy)))
        return None


def normalize_images(img_u8, mean=(0.485, 0.456, 0.406), std=(0.229, 0.224, 0.225)):
    """uint8 [B, 3, H, W] → NHWC with channels padded to 8 (bf16 on CUDA, fp32 on CPU)."""
    B, _, H, W = img_u8.shape
    if img_u8.is_cuda:
        out = torch.empty(B, H, W, 8, device=img_u8.device, dtype=torch.bfloat16)
        ic = img_u8 if img_u8.is_contiguous() else img_u8.contiguous()
        check(cuda_lib().nb_image_normalize(ptr(ic), ptr(out), ctypes.c_int(B), ctypes.c_int(H), ctypes.c_int(W),
                                            *(ctypes.c_float(v) for v in (*mean, *std)), stream_ptr()), "image_normalize")
        return out
    x = (img_u8.float() / 255.0 - torch.tensor(mean).view(1, 3, 1, 1)) / torch.tensor(std).view(1, 3, 1, 1)
    return torch.nn.functional.pad(x.permute(0, 2, 3, 1), (0, 5))
