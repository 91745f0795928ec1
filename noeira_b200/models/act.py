"""ACT (Action Chunking with Transformers): ResNet-18 backbone shared across cameras, CVAE encoder, DETR-style
post-LN encoder / decoder, L1 + KL loss.

Wiring follows the reference's loss graph (noeira/deep_agents/act/loss_graph.mojo:129-241) and layers
(layers.mojo:86-231): positions are added to queries and keys but not to values at EVERY layer; attention uses
four separate projections q / k / v / out; the decoder starts from LEARNED content queries ``tgt0`` (the
reference's deliberate deviation from the zero target) and its last layer feeds LayerNorm → Linear(ADIM).
Node names of the reference are kept as parameter prefixes: cls, qenc, aenc, cvae, latinfo, lattok, feat, src,
prop, addpos, memory, qpe, tgt0, hs, hsn, ahat.
Loss: L1 over valid chunk steps + kl_weight · KL(N(μ, σ²) ‖ N(0, 1)); AdamW lr 1e-5, wd 1e-4, batch 8 per GPU.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .. import nn
from ..nn.init import Normal
from ..nn.module import Module
from ..nn.transformer import AttentionCore


@dataclass
class ACTConfig:
    qpos_dim: int = 6
    action_dim: int = 6
    chunk: int = 100
    n_cam: int = 2
    height: int = 480
    width: int = 640
    dim: int = 512
    heads: int = 8
    ff: int = 3200
    enc_layers: int = 4
    dec_layers: int = 7
    latent: int = 32
    kl_weight: float = 10.0
    dropout: float = 0.1
    lr: float = 1e-5
    weight_decay: float = 1e-4
    seed: int = 0


def sinusoid_1d(n, d):
    pos = torch.arange(n, dtype=torch.float32)[:, None]
    i = torch.arange(d, dtype=torch.float32)[None, :]
    ang = pos / torch.pow(10000.0, 2 * torch.div(i, 2, rounding_mode="floor") / d)
    out = torch.zeros(n, d)
    out[:, 0::2] = ang[:, 0::2].sin()
    out[:, 1::2] = ang[:, 1::2].cos()
    return out


def sinusoid_2d(h, w, d):
    """DETR sine position embedding: half of the channels encode y, half x."""
    half = d // 2
    y = sinusoid_1d(h, half)[:, None, :].expand(h, w, half)
    x = sinusoid_1d(w, half)[None, :, :].expand(h, w, half)
    return torch.cat([y, x], -1).reshape(h * w, d)


class _MHA(Module):
    """Bare attention with four separate projections; positions are added by the caller."""

    def __init__(self, dim, heads):
        super().__init__()
        self.h, self.hd = heads, dim // heads
        self.q = self.add_child("q", nn.Linear(dim, dim))
        self.k = self.add_child("k", nn.Linear(dim, dim))
        self.v = self.add_child("v", nn.Linear(dim, dim))
        self.o = self.add_child("o", nn.Linear(dim, dim))
        self.core = AttentionCore()

    def forward(self, xq, xk, xv, key_valid=None):
        B, Sq, D = xq.shape
        Sk = xk.shape[1]
        q = self.q.forward(xq).reshape(B, Sq, self.h, self.hd)
        k = self.k.forward(xk).reshape(B, Sk, self.h, self.hd)
        v = self.v.forward(xv).reshape(B, Sk, self.h, self.hd)
        return self.o.forward(self.core.forward(q, k, v, key_valid=key_valid).reshape(B, Sq, D))

    def vjp(self, dy):
        B, Sq, D = dy.shape
        do = self.o.vjp(dy).reshape(B, Sq, self.h, self.hd)
        dq, dk, dv = self.core.vjp(do)
        Sk = dk.shape[1]
        return (self.q.vjp(dq.reshape(B, Sq, D)), self.k.vjp(dk.reshape(B, Sk, D)), self.v.vjp(dv.reshape(B, Sk, D)))


class _FFN(Module):
    def __init__(self, dim, ff, p):
        super().__init__()
        self.l1 = self.add_child("f1", nn.Linear(dim, ff, act="relu"))
        self.drop = self.add_child("drop", nn.Dropout(p))
        self.l2 = self.add_child("f2", nn.Linear(ff, dim))

    def forward(self, x):
        return self.l2.forward(self.drop.forward(self.l1.forward(x)))

    def vjp(self, dy):
        return self.l1.vjp(self.drop.vjp(self.l2.vjp(dy)))


class DETREncoderLayer(Module):
    """x = LN(x + Attn(q = k = x + pos, v = x));  x = LN(x + FFN(x))   (post-LN)."""

    def __init__(self, dim, heads, ff, p=0.1):
        super().__init__()
        self.attn = self.add_child("attn", _MHA(dim, heads))
        self.n1 = self.add_child("n1", nn.LayerNorm(dim))
        self.ffn = self.add_child("ffn", _FFN(dim, ff, p))
        self.n2 = self.add_child("out", nn.LayerNorm(dim))
        self.d1, self.d2 = self.add_child("d1", nn.Dropout(p)), self.add_child("d2", nn.Dropout(p))

    def forward(self, x, pos, key_valid=None):
        xp = x + pos
        n1 = self.n1.forward(x + self.d1.forward(self.attn.forward(xp, xp, x, key_valid)))
        return self.n2.forward(n1 + self.d2.forward(self.ffn.forward(n1)))

    def vjp(self, dy):
        dr2 = self.n2.vjp(dy)
        dn1 = dr2 + self.ffn.vjp(self.d2.vjp(dr2))
        dr1 = self.n1.vjp(dn1)
        dq, dk, dv = self.attn.vjp(self.d1.vjp(dr1))
        dxp = dq + dk
        return dr1 + dxp + dv, dxp


class DETRDecoderLayer(Module):
    def __init__(self, dim, heads, ff, p=0.1):
        super().__init__()
        self.sa = self.add_child("self", _MHA(dim, heads))
        self.n1 = self.add_child("n1", nn.LayerNorm(dim))
        self.ca = self.add_child("cross", _MHA(dim, heads))
        self.n2 = self.add_child("n2", nn.LayerNorm(dim))
        self.ffn = self.add_child("ffn", _FFN(dim, ff, p))
        self.n3 = self.add_child("out", nn.LayerNorm(dim))
        self.d1, self.d2, self.d3 = (self.add_child(f"d{i}", nn.Dropout(p)) for i in (1, 2, 3))

    def forward(self, x, qpos, kmem, mem):
        xq = x + qpos
        n1 = self.n1.forward(x + self.d1.forward(self.sa.forward(xq, xq, x)))
        n2 = self.n2.forward(n1 + self.d2.forward(self.ca.forward(n1 + qpos, kmem, mem)))
        return self.n3.forward(n2 + self.d3.forward(self.ffn.forward(n2)))

    def vjp(self, dy):
        dr3 = self.n3.vjp(dy)
        dn2 = dr3 + self.ffn.vjp(self.d3.vjp(dr3))
        dr2 = self.n2.vjp(dn2)
        dcq, dkmem, dmem = self.ca.vjp(self.d2.vjp(dr2))
        dn1 = dr2 + dcq
        dr1 = self.n1.vjp(dn1)
        dq, dk, dv = self.sa.vjp(self.d1.vjp(dr1))
        dxq = dq + dk
        return dr1 + dxq + dv, dxq + dcq, dkmem, dmem


class ACTModel(Module):
    def __init__(self, cfg: ACTConfig):
        super().__init__()
        self.cfg = cfg
        D, K = cfg.dim, cfg.chunk
        nn.manual_seed(cfg.seed)
        mk = lambda name, shape: self.add_param(name, shape, decay=False, init=Normal(0.0, 0.02))
        self.cls = mk("cls.queries", (1, D))
        self.qenc = self.add_child("qenc", nn.Linear(cfg.qpos_dim, D, need_input_grad=False))
        self.aenc = self.add_child("aenc", nn.Tokenwise(nn.Linear(cfg.action_dim, D, need_input_grad=False)))
        self.cvae = [self.add_child(f"cvae.{i}", DETREncoderLayer(D, cfg.heads, cfg.ff, cfg.dropout)) for i in range(cfg.enc_layers)]
        self.latinfo = self.add_child("latinfo", nn.Linear(D, 2 * cfg.latent, out_fp32=True))
        self.lattok = self.add_child("lattok", nn.Linear(cfg.latent, D))
        self.feat = self.add_child("feat", nn.Tokenwise(nn.ResNet18Backbone()))
        self.backbone = self.feat.inner
        self.src = self.add_child("src", nn.Tokenwise(nn.Linear(512, D)))
        self.prop = self.add_child("prop", nn.Linear(cfg.qpos_dim, D, need_input_grad=False))
        self.addpos = mk("addpos.queries", (2, D))
        self.memory = [self.add_child(f"memory.{i}", DETREncoderLayer(D, cfg.heads, cfg.ff, cfg.dropout)) for i in range(cfg.enc_layers)]
        self.qpe = mk("qpe.queries", (K, D))
        self.tgt0 = mk("tgt0.queries", (K, D))
        self.hs = [self.add_child(f"hs.{i}", DETRDecoderLayer(D, cfg.heads, cfg.ff, cfg.dropout)) for i in range(cfg.dec_layers)]
        self.hsn = self.add_child("hsn", nn.Tokenwise(nn.LayerNorm(D)))
        self.ahat = self.add_child("ahat", nn.Tokenwise(nn.Linear(D, cfg.action_dim, out_fp32=True)))
        self.oh, self.ow = math.ceil(cfg.height / 32), math.ceil(cfg.width / 32)
        self.ntok = cfg.n_cam * self.oh * self.ow
        self._pos_built = None

    def _build_pos(self, device, dt):
        if self._pos_built == (device, dt):
            return
        cfg = self.cfg
        self.epos = sinusoid_1d(cfg.chunk + 2, cfg.dim).to(device, dt)[None]
        self.impos = sinusoid_2d(self.oh, self.ow, cfg.dim).repeat(cfg.n_cam, 1).to(device, dt)
        self._pos_built = (device, dt)

    def _p(self, p, dt):
        return (p.shadow if self.on_cuda else p.data)[:, : p.shape[1]].to(dt)

    # ------------------------------------------------------------------
    def forward(self, qpos, images_u8, actions, enc_valid, eps):
        """qpos [B,Q] fp32, images uint8 [B, N_CAM, 3, H, W], actions [B,K,A], enc_valid [B,K+2] (1 = attend),
        eps [B, L] reparameterisation noise.  Returns (ahat [B,K,A] fp32, latinfo [B, 2L] fp32)."""
        cfg = self.cfg
        dev = qpos.device
        dt = torch.bfloat16 if self.on_cuda else torch.float32
        self._build_pos(dev, dt)
        B, K, D = qpos.shape[0], cfg.chunk, cfg.dim

        def pad8(t):
            if not self.on_cuda:
                return t.float()
            w = (t.shape[-1] + 7) // 8 * 8
            o = torch.zeros(*t.shape[:-1], w, device=dev, dtype=torch.bfloat16)
            o[..., : t.shape[-1]] = t
            return o[..., : t.shape[-1]]

        self._qpos, self._act = pad8(qpos), pad8(actions)
        # ---- CVAE encoder
        x = torch.cat([self._p(self.cls, dt)[None].expand(B, 1, D), self.qenc.forward(self._qpos)[:, None].to(dt),
                       self.aenc.forward(self._act).to(dt)], 1)
        for lyr in self.cvae:
            x = lyr.forward(x, self.epos, key_valid=enc_valid)
        self._cvae_out_shape = x.shape
        info = self.latinfo.forward(x[:, 0].contiguous())
        L = cfg.latent
        mu, logvar = info[:, :L].float(), info[:, L: 2 * L].float()
        self._eps, self._std = eps, (0.5 * logvar).exp()
        z = mu + self._std * eps
        lat = self.lattok.forward(pad8(z))
        return self._decode(lat, images_u8, B, dt), info.float()

    def infer(self, qpos, images_u8):
        """Deployment forward: the latent is the prior mean (z = 0; the reference runs the same graph with the CVAE
        branch multiplied by zero, noeira/deep_agents/act/loss_graph.mojo:44-53).  Returns the normalised chunk
        ``[B, K, A]`` fp32."""
        cfg = self.cfg
        dev = qpos.device
        dt = torch.bfloat16 if self.on_cuda else torch.float32
        self._build_pos(dev, dt)
        B = qpos.shape[0]
        q = qpos.float()
        if self.on_cuda:
            w = (q.shape[-1] + 7) // 8 * 8
            o = torch.zeros(B, w, device=dev, dtype=torch.bfloat16)
            o[:, : q.shape[-1]] = q
            q = o[:, : q.shape[-1]]
        self._qpos = q
        zw = (cfg.latent + 7) // 8 * 8 if self.on_cuda else cfg.latent
        z = torch.zeros(B, zw, device=dev, dtype=dt)[:, : cfg.latent]
        lat = self.lattok.forward(z)
        return self._decode(lat, images_u8, B, dt)

    def _decode(self, lat, images_u8, B, dt):
        cfg = self.cfg
        K, D = cfg.chunk, cfg.dim
        # ---- vision
        imgs = nn.normalize_images(images_u8.reshape(B * cfg.n_cam, 3, cfg.height, cfg.width))
        f = self.backbone.forward(imgs)                                  # [B·NC, oh, ow, 512]
        self._fshape = f.shape
        src = self.src.forward(f.reshape(B, self.ntok, 512))
        mem = torch.cat([lat[:, None].to(dt), self.prop.forward(self._qpos)[:, None].to(dt), src.to(dt)], 1)
        mpos = torch.cat([self._p(self.addpos, dt), self.impos], 0)[None]
        self._mpos = mpos
        for lyr in self.memory:
            mem = lyr.forward(mem, mpos)
        # ---- decoder
        kmem = mem + mpos
        qpe = self._p(self.qpe, dt)[None]
        h = self._p(self.tgt0, dt)[None].expand(B, K, D).contiguous()
        for lyr in self.hs:
            h = lyr.forward(h, qpe, kmem, mem)
        ahat = self.ahat.forward(self.hsn.forward(h))
        return ahat.float()

    def vjp(self, dahat, dinfo_kl):
        """dahat [B,K,A] and the KL gradient wrt latinfo [B, 2L]; accumulates every parameter gradient."""
        cfg = self.cfg
        B, K, D, L = dahat.shape[0], cfg.chunk, cfg.dim, cfg.latent
        cast = (lambda t: t.to(torch.bfloat16)) if self.on_cuda else (lambda t: t.float())

        def padg(t):
            if not self.on_cuda:
                return t
            w = (t.shape[-1] + 7) // 8 * 8
            o = torch.zeros(*t.shape[:-1], w, device=t.device, dtype=torch.bfloat16)
            o[..., : t.shape[-1]] = t
            return o[..., : t.shape[-1]]

        dh = self.hsn.vjp(self.ahat.vjp(padg(cast(dahat))))
        dqpe = dkmem = dmem = None
        for lyr in reversed(self.hs):
            dh, g_qpe, g_kmem, g_mem = lyr.vjp(dh)
            dqpe = g_qpe if dqpe is None else dqpe + g_qpe
            dkmem = g_kmem if dkmem is None else dkmem + g_kmem
            dmem = g_mem if dmem is None else dmem + g_mem
        self.tgt0.grad.add_(dh.float().sum(0))
        self.qpe.grad.add_(dqpe.float().sum(0))
        dm = dmem + dkmem
        dmpos = dkmem.float().sum(0)
        for lyr in reversed(self.memory):
            dm, g_pos = lyr.vjp(dm)
            dmpos = dmpos + g_pos.float().sum(0)
        self.addpos.grad.add_(dmpos[:2])
        dlat, dprop, dsrc = dm[:, 0], dm[:, 1], dm[:, 2:]
        self.prop.vjp(dprop.contiguous())
        df = self.src.vjp(dsrc.contiguous())
        self.backbone.vjp(df.reshape(self._fshape))
        dz = self.lattok.vjp(dlat.contiguous()).float()[:, :L]
        dinfo = torch.cat([dz, dz * self._eps * self._std * 0.5], 1) + dinfo_kl.float()
        dcls = self.latinfo.vjp(padg(cast(dinfo)))
        dx = torch.zeros(self._cvae_out_shape, device=dahat.device, dtype=dcls.dtype)
        dx[:, 0] = dcls
        for lyr in reversed(self.cvae):
            dx, _ = lyr.vjp(dx)
        self.cls.grad.add_(dx[:, 0].float().sum(0, keepdim=True))
        self.qenc.vjp(dx[:, 1].contiguous())
        self.aenc.vjp(dx[:, 2:].contiguous())


class ACTTrainer:
    """train_step(batch) → device loss accumulators; one AdamW arena, optional fused DDP gradient sync
    (noeira/deep_agents/act/trainer.mojo:383,883-913)."""

    def __init__(self, cfg: ACTConfig = None, device="cuda", grad_sync=None):
        self.cfg = cfg = cfg or ACTConfig()
        self.device = torch.device(device)
        self.model = ACTModel(cfg).to(self.device)
        self.opt = nn.AdamW(self.model.named_params(), lr=cfg.lr, weight_decay=cfg.weight_decay)
        self.grad_sync = grad_sync
        if grad_sync is not None:
            grad_sync.attach(self.opt)
        self.loss_acc = torch.zeros(2, device=self.device)   # [l1, kl]
        self.gen = torch.Generator(device=self.device).manual_seed(cfg.seed + 11)
        self.l1 = nn.MSELoss(l1=True)
        self._graphed = None

    def step(self, qpos, images_u8, actions, enc_valid):
        """One optimisation step replayed from a CUDA graph (captured on the third call; shapes must stay fixed)."""
        if self._graphed is None:
            from ..utils.graphs import GraphedStep
            self._graphed = GraphedStep(self.train_step, [qpos, images_u8, actions, enc_valid], generators=[self.gen])
        return self._graphed(qpos, images_u8, actions, enc_valid)

    def train_step(self, qpos, images_u8, actions, enc_valid):
        cfg = self.cfg
        B = qpos.shape[0]
        nn.advance_rng(self.device)
        eps = torch.randn(B, cfg.latent, device=self.device, generator=self.gen)
        ahat, info = self.model.forward(qpos, images_u8, actions, enc_valid, eps)
        valid = enc_valid[:, 2:].float()
        n_valid = valid.sum().clamp_min(1.0)
        diff = (ahat - actions.float()) * valid[..., None]
        self.loss_acc[0] += diff.abs().sum() / (n_valid * cfg.action_dim)
        dahat = torch.sign(diff) / (n_valid * cfg.action_dim)
        L = cfg.latent
        mu, logvar = info[:, :L], info[:, L:]
        self.loss_acc[1] += (-0.5 * (1 + logvar - mu * mu - logvar.exp())).sum(1).mean()
        dinfo = torch.cat([mu, 0.5 * (logvar.exp() - 1)], 1) * (cfg.kl_weight / B)
        self.model.vjp(dahat, dinfo)
        if self.grad_sync is not None:
            self.grad_sync.reduce_and_step(self.opt)
        else:
            self.opt.step(zero_grad=True)
        return self.loss_acc
