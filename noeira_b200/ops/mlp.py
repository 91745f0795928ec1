"""Fused three-layer MLP kernels (``csrc/mlp_fused_tcgen05.cu``) for Linear+act → Linear+act → Linear with hidden width
256, input width <= 64 and output width <= 16 — the actor / critic shape of the RL trainers.

* ``mlp3_forward`` / ``mlp3_forward_group``: the whole forward in one launch (two networks: still one launch).
* ``mlp3_backward_group``: the data-gradient chain g2 = (dy W3ᵀ)⊙f'(h2), g1 = (g2 W2ᵀ)⊙f'(h1) in one launch.
* ``mlp3_param_grads``: the six weight-gradient GEMMs (split-K into the fp32 gradient arena) and bias column sums of
  a network, each layer on its own side stream so they overlap.
Reference shapes: noeira/deep_agents/ppo/trainer.mojo:837-915 (actor / critic update of PPO).
"""
from __future__ import annotations

import ctypes

import torch

from .._native import check, cuda_lib, ptr, stream_ptr
from .gemm import ACT
from .status import device_status


class NbMlpNet(ctypes.Structure):
    """Mirror of ``struct NbMlpNet`` (csrc/mlp_fused_tcgen05.cu): same field order."""
    _fields_ = ([(n, ctypes.c_void_p) for n in ("x", "w1", "w2", "w3", "b1", "b2", "b3", "out", "h1", "h2", "dy", "g1", "g2",
                                                 "bias_part", "db1", "db2", "db3")]
                + [(n, ctypes.c_int) for n in ("ldx", "ldw1", "ldw2", "ldw3", "ld_out", "ld_h", "ld_dy", "ld_g", "M", "k0", "n3",
                                               "act")])


def fusable(l1, l2, l3) -> bool:
    return (l1.on_cuda and l1.out_dim == 256 and l2.in_dim == 256 and l2.out_dim == 256 and l3.in_dim == 256
            and l1.in_dim <= 64 and l3.out_dim <= 16 and l1.act == l2.act and l1.act in ("tanh", "relu") and l3.act is None
            and l1.bias is not None and l2.bias is not None)


def _p(t):
    return t.data_ptr() if t is not None else None


class Mlp3Pass:
    """Buffers of one network for a fused forward (+ backward) over ``M`` rows; reusable across steps (stable addresses
    for CUDA-graph capture)."""

    def __init__(self, l1, l2, l3, M: int, device, train: bool = True):
        self.l1, self.l2, self.l3, self.M = l1, l2, l3, M
        f = dict(device=device, dtype=torch.float32)
        h = dict(device=device, dtype=torch.bfloat16)
        self.out = torch.empty(M, 16, **f)
        self.h1 = torch.empty(M, 256, **h) if train else None
        self.h2 = torch.empty(M, 256, **h) if train else None
        self.g1 = torch.empty(M, 256, **h) if train else None
        self.g2 = torch.empty(M, 256, **h) if train else None
        # per-CTA column sums of g1, g2, dy: the bias gradients come out of the data-gradient kernel
        self.bias_part = torch.empty((M + 127) // 128, 3, 256, **f) if train else None

    def net(self, x, dy=None) -> NbMlpNet:
        l1, l2, l3 = self.l1, self.l2, self.l3
        w1, w2, w3 = l1.weight.shadow, l2.weight.shadow, l3.weight.shadow
        n = NbMlpNet()
        n.x, n.w1, n.w2, n.w3 = x.data_ptr(), w1.data_ptr(), w2.data_ptr(), w3.data_ptr()
        n.b1, n.b2, n.b3 = l1.bias.storage.data_ptr(), l2.bias.storage.data_ptr(), _p(l3.bias.storage if l3.bias is not None else None)
        n.out, n.h1, n.h2 = self.out.data_ptr(), _p(self.h1), _p(self.h2)
        n.dy, n.g1, n.g2 = _p(dy), _p(self.g1), _p(self.g2)
        if dy is not None:
            n.bias_part = _p(self.bias_part)
            n.db1, n.db2 = l1.bias.grad_storage.data_ptr(), l2.bias.grad_storage.data_ptr()
            n.db3 = _p(l3.bias.grad_storage if l3.bias is not None else None)
        n.ldx, n.ldw1, n.ldw2, n.ldw3 = x.stride(0), w1.stride(0), w2.stride(0), w3.stride(0)
        n.ld_out, n.ld_h, n.ld_g = 16, 256, 256
        n.ld_dy = dy.stride(0) if dy is not None else 0
        n.M, n.k0, n.n3, n.act = x.shape[0], l1.in_dim, l3.out_dim, ACT[l1.act]
        return n

    @property
    def y(self):
        return self.out[:, : self.l3.out_dim]


def mlp3_forward_group(passes, xs):
    """Forward of one or two networks (``Mlp3Pass`` each) on inputs ``xs`` (bf16 ``[M, >= in_dim]``, 16-byte row
    pitch) in ONE launch.  Returns the fp32 outputs ``[M, out_dim]``."""
    arr = (NbMlpNet * len(passes))(*[p.net(x[:, : p.l1.in_dim]) for p, x in zip(passes, xs)])
    check(cuda_lib().nb_mlp3_fwd_group(arr, ctypes.c_int(len(passes)), ptr(device_status(xs[0].device)), stream_ptr()),
          "mlp3_fwd_group")
    return [p.y for p in passes]


def mlp3_backward_group(passes, xs, dys):
    """Data-gradient chain of one or two networks in ONE launch; fills ``pass.g1`` / ``pass.g2`` (gradients of the
    pre-activations of layers 1 and 2) and ACCUMULATES the three bias gradients of each network (column sums of g1,
    g2, dy: per-CTA partials from the same kernel, added in CTA order by a second small launch).
    ``dys``: bf16 ``[M, >= out_dim]`` with a 16-byte row pitch."""
    arr = (NbMlpNet * len(passes))(*[p.net(x[:, : p.l1.in_dim], dy) for p, x, dy in zip(passes, xs, dys)])
    check(cuda_lib().nb_mlp3_bwd_group(arr, ctypes.c_int(len(passes)), ptr(device_status(xs[0].device)), stream_ptr()),
          "mlp3_bwd_group")


def mlp3_param_grads(p: Mlp3Pass, x, dy, branches=None):
    """dW3 += h2ᵀ dy, dW2 += h1ᵀ g2, dW1 += xᵀ g1, accumulated into the parameters' fp32 gradient storage (the bias
    gradients were produced by ``mlp3_backward_group``).  ``branches``: three ``ops.streams.Branch`` objects, one per
    layer, so the three split-K GEMMs overlap; the caller joins them before the optimizer step."""
    from .. import ops
    work = ((p.l3, p.h2, dy), (p.l2, p.h1, p.g2), (p.l1, x[:, : p.l1.in_dim], p.g1))
    for i, (lin, a, g) in enumerate(work):
        n = lin.out_dim

        def run(lin=lin, a=a, g=g, n=n):
            ops.gemm(a, g[:, :n], a_mn=True, b_mn=True, out=lin.weight.grad_storage, accumulate=True, n=n)
        if branches is not None:
            with branches[i]:
                run()
        else:
            run()


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
