"""GPT-style decoder language models and a ViT classifier built from the framework's leaves.

``GPT(vocab, seq, dim, layers, heads)``: token + learned position embeddings, pre-norm causal transformer blocks
(packed-QKV flash attention, GELU feed-forward), final LayerNorm, untied or tied output projection.  ``dropout`` adds
counter-hash dropout after the embeddings and inside every block residual branch (GPTDrop); ``tie=True`` shares the
embedding matrix with the head (GPTDropTied).  Residual output projections are initialised with std 0.02/sqrt(2L)
(``gpt_scale_residual_proj``).  Parameter names follow the child paths: ``wte.weight``, ``wpe.weight``,
``blocks.<i>.norm1.gamma`` …, ``ln_f.gamma``, ``head.weight``.
Reference: noeira/nn/models/gpt.mojo:75,159,193,267,316; ViT / PatchEmbed noeira/nn/models/vit.mojo:25,41.
"""
from __future__ import annotations

import math

import torch

from .. import nn
from ..nn.module import Module


class GPT(Module):
    def __init__(self, vocab: int, seq: int, dim: int = 384, layers: int = 6, heads: int = 6, ff_mult: int = 4,
                 dropout: float = 0.0, tie: bool = False, seed: int = 0):
        super().__init__()
        nn.manual_seed(seed)
        self.vocab, self.seq, self.dim, self.tie = vocab, seq, dim, tie
        self.wte = self.add_child("wte", nn.Embedding(vocab, dim))
        self.wpe = self.add_child("wpe", nn.Embedding(seq, dim))
        self.drop = self.add_child("drop", nn.Dropout(dropout)) if dropout > 0 else None
        self.blocks = [self.add_child(f"blocks.{i}", nn.TransformerBlock(dim, heads, ff_mult * dim, norm="layer", ffn="gelu",
                                                                         mask="causal")) for i in range(layers)]
        self.block_drop = [(self.add_child(f"drop_a.{i}", nn.Dropout(dropout)), self.add_child(f"drop_f.{i}", nn.Dropout(dropout)))
                           for i in range(layers)] if dropout > 0 else None
        self.ln_f = self.add_child("ln_f", nn.LayerNorm(dim))
        self.head = None if tie else self.add_child("head", nn.Linear(dim, vocab, bias=False, out_fp32=False))
        # residual projections scaled by 1/sqrt(2L)
        s = 1.0 / math.sqrt(2 * layers)
        for b in self.blocks:
            for lin in (b.attn.out, b.ffn.l1):
                lin.weight.data.mul_(s)
                lin.weight.version += 1

    def forward(self, ids: torch.Tensor):
        """ids int64 [B, S] → logits [B, S, vocab] (bf16 on CUDA)."""
        B, S = ids.shape
        self._shape = (B, S)
        pos = torch.arange(S, device=ids.device).expand(B, S)
        x = self.wte.forward(ids) + self.wpe.forward(pos)
        if self.drop is not None:
            x = self.drop.forward(x)
        for b in self.blocks:
            x = b.forward(x)
        h = self.ln_f.forward(x)
        self._h = h
        if self.tie:
            W = self.wte.weight
            if h.is_cuda:
                from ..ops.gemm import gemm
                logits = gemm(h.reshape(B * S, self.dim), W.shadow[:, : self.dim])      # h @ Eᵀ: E is [vocab, dim] = [N, K]
                return logits.reshape(B, S, -1)[..., : self.vocab]
            return h.float() @ W.data.t()
        return self.head.forward(h)

    def vjp(self, dlogits):
        B, S = self._shape
        if self.tie:
            W = self.wte.weight
            d2 = dlogits.reshape(B * S, -1)
            if dlogits.is_cuda:
                from ..ops.gemm import gemm
                h2 = self._h.reshape(B * S, self.dim)
                d2 = d2 if d2.dtype == torch.bfloat16 else d2.to(torch.bfloat16)
                gemm(d2, h2, a_mn=True, b_mn=True, out=W.grad_storage, accumulate=True, n=self.dim)   # dE += dlogitsᵀ h
                dh = gemm(d2, W.shadow[:, : self.dim], b_mn=True).reshape(B, S, self.dim)              # dlogits @ E
            else:
                W.grad.add_(d2.float().t() @ self._h.reshape(B * S, self.dim).float())
                dh = (d2.float() @ W.data).reshape(B, S, self.dim)
        else:
            dh = self.head.vjp(dlogits)
        dx = self.ln_f.vjp(dh)
        for b in reversed(self.blocks):
            dx = b.vjp(dx)
        if self.drop is not None:
            dx = self.drop.vjp(dx)
        self.wte.vjp(dx)
        self.wpe.vjp(dx)
        return None


class PatchEmbed(Module):
    """[B, 3, H, W] → [B, (H/p)(W/p), dim]: non-overlapping patches through one Linear (= a stride-p convolution)."""

    def __init__(self, image: int, patch: int, dim: int, channels: int = 3):
        super().__init__()
        self.image, self.patch, self.channels = image, patch, channels
        self.proj = self.add_child("proj", nn.Linear(channels * patch * patch, dim, need_input_grad=False))

    def forward(self, img):
        B, g, p, c = img.shape[0], self.image // self.patch, self.patch, self.channels
        dt = torch.bfloat16 if self.on_cuda else torch.float32
        x = img.to(dt).reshape(B, c, g, p, g, p).permute(0, 2, 4, 1, 3, 5).reshape(B, g * g, c * p * p)
        return self.proj.forward(x.contiguous())

    def vjp(self, dy):
        self.proj.vjp(dy)
        return None


class ViT(Module):
    """Patch embedding + class token + learned positions + pre-norm encoder blocks + LayerNorm + linear classifier."""

    def __init__(self, image: int = 32, patch: int = 4, dim: int = 192, layers: int = 6, heads: int = 3, classes: int = 10,
                 ff_mult: int = 4, seed: int = 0):
        super().__init__()
        nn.manual_seed(seed)
        self.dim = dim
        n = (image // patch) ** 2
        self.embed = self.add_child("patch_embed", PatchEmbed(image, patch, dim))
        self.cls = self.add_param("cls_token", (1, dim), decay=False, init=nn.Normal(0, 0.02))
        self.pos = self.add_param("pos_embed", (n + 1, dim), decay=False, init=nn.Normal(0, 0.02))
        self.blocks = [self.add_child(f"blocks.{i}", nn.TransformerBlock(dim, heads, ff_mult * dim)) for i in range(layers)]
        self.norm = self.add_child("norm", nn.LayerNorm(dim))
        self.head = self.add_child("head", nn.Linear(dim, classes, out_fp32=True))

    def _p(self, p):
        return (p.shadow if self.on_cuda else p.data)[:, : self.dim]

    def forward(self, img):
        x = self.embed.forward(img)
        B = x.shape[0]
        x = torch.cat([self._p(self.cls).to(x.dtype).expand(B, 1, self.dim), x], 1) + self._p(self.pos).to(x.dtype)[None]
        x = x.contiguous()
        for b in self.blocks:
            x = b.forward(x)
        h = self.norm.forward(x)
        self._tokens = h.shape[1]
        return self.head.forward(h[:, 0].contiguous())

    def vjp(self, dlogits):
        dcls = self.head.vjp(dlogits)
        B = dcls.shape[0]
        dh = torch.zeros(B, self._tokens, self.dim, device=dcls.device, dtype=dcls.dtype)
        dh[:, 0] = dcls
        dx = self.norm.vjp(dh)
        for b in reversed(self.blocks):
            dx = b.vjp(dx)
        self.pos.grad[:, : self.dim].add_(dx.float().sum(0))
        self.cls.grad[:, : self.dim].add_(dx[:, 0].float().sum(0, keepdim=True))
        self.embed.vjp(dx[:, 1:].contiguous())
        return None
