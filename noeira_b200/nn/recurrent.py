"""Recurrent cells with explicit backward: ``GRUCell``, ``LSTMCell`` and ``LSTMSeq`` (unrolled over time with stored gate
activations), built on ``Linear`` so the gate GEMMs run on the tcgen05 kernel on CUDA.  Gate order and parameter names
follow the reference (noeira/nn/primitives/gru_cell.mojo, lstm_cell.mojo, lstm_seq.mojo): children ``ih`` (input →
gates) and ``hh`` (hidden → gates); GRU gates ``[r | z | n]``, LSTM gates ``[i | f | g | o]``.
"""
from __future__ import annotations

import torch

from .layers import Linear
from .module import Module


class GRUCell(Module):
    ARITY = 2

    def __init__(self, in_dim: int, hidden: int):
        super().__init__()
        self.hidden = hidden
        self.ih = self.add_child("ih", Linear(in_dim, 3 * hidden))
        self.hh = self.add_child("hh", Linear(hidden, 3 * hidden))

    def forward(self, x, h):
        H = self.hidden
        gi, gh = self.ih.forward(x).float(), self.hh.forward(h).float()
        r = torch.sigmoid(gi[:, :H] + gh[:, :H])
        z = torch.sigmoid(gi[:, H:2 * H] + gh[:, H:2 * H])
        n = torch.tanh(gi[:, 2 * H:] + r * gh[:, 2 * H:])
        hf = h.float()
        self._c = (r, z, n, gh[:, 2 * H:], hf)
        return ((1 - z) * n + z * hf).to(h.dtype)

    def vjp(self, dh_new):
        r, z, n, ghn, h = self._c
        d = dh_new.float()
        dn = d * (1 - z)
        dz = d * (h - n)
        dpre_n = dn * (1 - n * n)
        dr = dpre_n * ghn
        dpre_r, dpre_z = dr * r * (1 - r), dz * z * (1 - z)
        dgi = torch.cat([dpre_r, dpre_z, dpre_n], 1)
        dgh = torch.cat([dpre_r, dpre_z, dpre_n * r], 1)
        dt = dh_new.dtype
        dx = self.ih.vjp(dgi.to(dt))
        dh = self.hh.vjp(dgh.to(dt)).float() + d * z
        return dx, dh.to(dt)


class LSTMCell(Module):
    ARITY = 3

    def __init__(self, in_dim: int, hidden: int):
        super().__init__()
        self.hidden = hidden
        self.ih = self.add_child("ih", Linear(in_dim, 4 * hidden))
        self.hh = self.add_child("hh", Linear(hidden, 4 * hidden, bias=False))

    def forward(self, x, h, c):
        H = self.hidden
        g = self.ih.forward(x).float() + self.hh.forward(h).float()
        i, f, gg, o = torch.sigmoid(g[:, :H]), torch.sigmoid(g[:, H:2 * H]), torch.tanh(g[:, 2 * H:3 * H]), torch.sigmoid(g[:, 3 * H:])
        c2 = f * c.float() + i * gg
        tc = torch.tanh(c2)
        self._c = (i, f, gg, o, c.float(), tc)
        return (o * tc).to(h.dtype), c2.to(c.dtype)

    def vjp(self, dh, dc):
        i, f, gg, o, c, tc = self._c
        dhf = dh.float()
        dc2 = (dc.float() if dc is not None else 0) + dhf * o * (1 - tc * tc)
        dg = torch.cat([dc2 * gg * i * (1 - i), dc2 * c * f * (1 - f), dc2 * i * (1 - gg * gg), dhf * tc * o * (1 - o)], 1).to(dh.dtype)
        dx = self.ih.vjp(dg)
        dhp = self.hh.vjp(dg)
        return dx, dhp, (dc2 * f).to(dh.dtype)


class LSTMSeq(Module):
    """``x [B, T, in]`` → ``h [B, T, hidden]``; one cell instance per time step shares the parameters (the per-step caches
    are kept in a list so the backward can walk the sequence in reverse)."""

    def __init__(self, in_dim: int, hidden: int):
        super().__init__()
        self.hidden = hidden
        self.cell = self.add_child("cell", LSTMCell(in_dim, hidden))

    def forward(self, x, h0=None, c0=None):
        B, T, _ = x.shape
        h = h0 if h0 is not None else torch.zeros(B, self.hidden, device=x.device, dtype=x.dtype)
        c = c0 if c0 is not None else torch.zeros(B, self.hidden, device=x.device, dtype=x.dtype)
        self._steps, out = [], []
        for t in range(T):
            h, c = self.cell.forward(x[:, t].contiguous(), h, c)
            self._steps.append((self.cell._c, self.cell.ih._x, self.cell.ih._saved, self.cell.hh._x, self.cell.hh._saved))
            out.append(h)
        return torch.stack(out, 1)

    def vjp(self, dout):
        B, T, _ = dout.shape
        dh = torch.zeros(B, self.hidden, device=dout.device, dtype=dout.dtype)
        dc = torch.zeros(B, self.hidden, device=dout.device, dtype=dout.dtype)
        dxs = [None] * T
        for t in reversed(range(T)):
            (self.cell._c, self.cell.ih._x, self.cell.ih._saved, self.cell.hh._x, self.cell.hh._saved) = self._steps[t]
            dxs[t], dh, dc = self.cell.vjp(dout[:, t] + dh, dc)
        return torch.stack(dxs, 1)
