"""SmolVLA-style flow-matching vision-language-action model.

  vision   12-layer ViT (d 768, 12 heads, FF 3072, patch 16, 512² → 1024 tokens) → pixel shuffle (×4 → 64 tokens
           of 12288) → connector Linear(12288 → 960), scaled by √960
  language 16-layer decoder (hidden 960, 15 query / 5 KV heads of 64, SwiGLU FF 2560, RMSNorm, RoPE θ = 1e5,
           vocab 49152) over the prefix [images… | language ids | state token]; prefix-LM block mask: images and
           language attend each other bidirectionally, the state token attends everything
  expert   16 layers of width 720 (queries in the VLM head geometry 15×64, KV width 320, FF 2048): even layers
           self-attend over [prefix K/V of the same VLM layer ; suffix] (suffix causal), odd layers cross-attend
           the prefix K/V; suffix = per-token concat [action embedding ‖ sinusoidal time embedding] → MLP
  loss     flow matching: t ~ Beta(1.5, 1)·0.999 + 0.001, x_t = t·noise + (1−t)·actions, target u = noise − actions,
           MSE over the real action columns; inference = 10 Euler steps from t = 1 to 0 with dt = −0.1.

Training follows the reference's fine-tune step: the prefix (vision + language) is computed once without
gradient (frozen), the expert and the action / time / state projections are trained
(noeira/deep_agents/smolvla/train_step.mojo:1-40, expert.mojo:7-35,68-73, flow_loss.mojo:1-104, attn_mask.mojo:80-105).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .. import nn
from ..nn.module import Module
from ..nn.transformer import AttentionCore, rope_


@dataclass
class VLAConfig:
    image: int = 512
    patch: int = 16
    n_cam: int = 3
    vit_dim: int = 768
    vit_heads: int = 12
    vit_ff: int = 3072
    vit_layers: int = 12
    shuffle: int = 4
    hidden: int = 960
    heads: int = 15
    kv_heads: int = 5
    head_dim: int = 64
    ff: int = 2560
    lm_layers: int = 16
    vocab: int = 49152
    n_lang: int = 48
    expert_width: int = 720
    expert_ff: int = 2048
    chunk: int = 50
    action_dim: int = 6
    action_pad: int = 32
    rope_theta: float = 1e5
    lr: float = 1e-4
    seed: int = 0

    @property
    def tokens_per_image(self):
        return (self.image // self.patch // self.shuffle) ** 2

    @property
    def prefix_len(self):
        return self.n_cam * self.tokens_per_image + self.n_lang + 1


class VisionTower(Module):
    def __init__(self, c: VLAConfig):
        super().__init__()
        self.c = c
        pd = 3 * c.patch * c.patch
        self.patch = self.add_child("patch_embed", nn.Linear(pd, c.vit_dim))
        n = (c.image // c.patch) ** 2
        self.pos = self.add_param("pos_embed", (n, c.vit_dim), decay=False, init=nn.Normal(0, 0.02))
        self.blocks = [self.add_child(f"layers.{i}", nn.TransformerBlock(c.vit_dim, c.vit_heads, c.vit_ff, norm="layer",
                                                                          ffn="gelu", eps=1e-6)) for i in range(c.vit_layers)]
        self.norm = self.add_child("post_norm", nn.LayerNorm(c.vit_dim, 1e-6))
        self.connector = self.add_child("connector", nn.Linear(c.vit_dim * c.shuffle ** 2, c.hidden, bias=False))

    def forward(self, img):
        """img [N, 3, H, W] in [0, 1] → [N, tokens_per_image, hidden]"""
        c = self.c
        N = img.shape[0]
        g = c.image // c.patch
        dt = torch.bfloat16 if self.on_cuda else torch.float32
        p = img.to(dt).reshape(N, 3, g, c.patch, g, c.patch).permute(0, 2, 4, 1, 3, 5).reshape(N, g * g, 3 * c.patch * c.patch)
        x = self.patch.forward(p.contiguous()).to(dt)
        pos = (self.pos.shadow if self.on_cuda else self.pos.data)[:, : c.vit_dim].to(dt)
        x = x + pos[None]
        for b in self.blocks:
            x = b.forward(x)
            b.release_buffers()
        x = self.norm.forward(x)
        s = c.shuffle
        x = x.reshape(N, g // s, s, g // s, s, c.vit_dim).permute(0, 1, 3, 2, 4, 5).reshape(N, (g // s) ** 2, s * s * c.vit_dim)
        return self.connector.forward(x.contiguous()) * math.sqrt(c.hidden)


class ExpertLayer(Module):
    def __init__(self, c: VLAConfig, cross: bool):
        super().__init__()
        W, QW, KVW = c.expert_width, c.heads * c.head_dim, c.kv_heads * c.head_dim
        self.c, self.cross = c, cross
        self.n1 = self.add_child("input_layernorm", nn.RMSNorm(W))
        self.q = self.add_child("self_attn.q_proj", nn.Linear(W, QW, bias=False))
        self.k = self.add_child("self_attn.k_proj", nn.Linear(KVW if cross else W, KVW, bias=False, need_input_grad=not cross))
        self.v = self.add_child("self_attn.v_proj", nn.Linear(KVW if cross else W, KVW, bias=False, need_input_grad=not cross))
        self.o = self.add_child("self_attn.o_proj", nn.Linear(QW, W, bias=False))
        self.n2 = self.add_child("post_attention_layernorm", nn.RMSNorm(W))
        self.mlp = self.add_child("mlp", nn.SwiGLUFFN(W, c.expert_ff, bias=False))
        self.core = AttentionCore(mask=None if cross else "causal")

    def forward(self, x, pk, pv, P):
        """x [B, S, W]; pk/pv: prefix keys / values [B, P, 5, 64] of the matching VLM layer (no gradient)."""
        c = self.c
        B, S, _ = x.shape
        h = self.n1.forward(x)
        q = self.q.forward(h).reshape(B, S, c.heads, c.head_dim)
        rope_(q, c.rope_theta, pos0=P)
        if self.cross:
            flat = torch.cat([pk.reshape(B, P, -1), pv.reshape(B, P, -1)], 0)      # project the cached prefix K/V
            k = self.k.forward(flat[:B].contiguous()).reshape(B, P, c.kv_heads, c.head_dim)
            v = self.v.forward(flat[B:].contiguous()).reshape(B, P, c.kv_heads, c.head_dim)
            self.core.causal_off = 0
        else:
            ks = self.k.forward(h).reshape(B, S, c.kv_heads, c.head_dim)
            vs = self.v.forward(h).reshape(B, S, c.kv_heads, c.head_dim)
            rope_(ks, c.rope_theta, pos0=P)
            k = torch.cat([pk, ks.to(pk.dtype)], 1)
            v = torch.cat([pv, vs.to(pv.dtype)], 1)
            self.core.causal_off = P             # suffix token i sees the whole prefix and suffix tokens <= i
        a = self.core.forward(q, k.contiguous(), v.contiguous())
        x = x + self.o.forward(a.reshape(B, S, c.heads * c.head_dim))
        self._P, self._S = P, S
        return x + self.mlp.forward(self.n2.forward(x))

    def vjp(self, dy):
        c, P, S = self.c, self._P, self._S
        B = dy.shape[0]
        d = dy + self.n2.vjp(self.mlp.vjp(dy))
        da = self.o.vjp(d).reshape(B, S, c.heads, c.head_dim)
        dq, dk, dv = self.core.vjp(da)
        rope_(dq, c.rope_theta, pos0=P, backward=True)
        dh = self.q.vjp(dq.reshape(B, S, -1))
        if self.cross:
            self.k.vjp(dk.reshape(B, P, -1))
            self.v.vjp(dv.reshape(B, P, -1))
        else:
            dks, dvs = dk[:, P:].contiguous(), dv[:, P:].contiguous()
            rope_(dks, c.rope_theta, pos0=P, backward=True)
            dh = dh + self.k.vjp(dks.reshape(B, S, -1)) + self.v.vjp(dvs.reshape(B, S, -1))
        return d + self.n1.vjp(dh)


class VLAModel(Module):
    def __init__(self, c: VLAConfig):
        super().__init__()
        self.c = c
        nn.manual_seed(c.seed)
        self.vision = self.add_child("vision_model", VisionTower(c))
        self.embed = self.add_child("text_model.embed_tokens", nn.Embedding(c.vocab, c.hidden))
        self.lm = [self.add_child(f"text_model.layers.{i}", nn.TransformerBlock(
            c.hidden, c.heads, c.ff, kv_heads=c.kv_heads, head_dim=c.head_dim, norm="rms", ffn="swiglu",
            rope_theta=c.rope_theta, bias=False)) for i in range(c.lm_layers)]
        self.state_proj = self.add_child("state_proj", nn.Linear(c.action_pad, c.hidden))
        self.action_in = self.add_child("action_in_proj", nn.Linear(c.action_pad, c.expert_width))
        self.time_in = self.add_child("action_time_mlp_in", nn.Linear(2 * c.expert_width, c.expert_width, act="silu"))
        self.time_out = self.add_child("action_time_mlp_out", nn.Linear(c.expert_width, c.expert_width))
        self.expert = [self.add_child(f"lm_expert.layers.{i}", ExpertLayer(c, cross=(i % 2 == 1))) for i in range(c.lm_layers)]
        self.expert_norm = self.add_child("lm_expert.norm", nn.RMSNorm(c.expert_width))
        self.action_out = self.add_child("action_out_proj", nn.Linear(c.expert_width, c.action_pad, out_fp32=True))
        self._mask = None

    def trainable(self):
        """Expert-only fine-tune: the vision tower, the language tower and the token embedding stay frozen."""
        frozen = ("vision_model.", "text_model.")
        return [(n, p) for n, p in self.named_params() if not n.startswith(frozen)]

    def prefix_mask(self, device):
        P = self.c.prefix_len
        if self._mask is None or self._mask.device != device:
            m = torch.zeros(P, P, device=device)
            m[: P - 1, P - 1] = float("-inf")       # nobody but the state token itself sees the state token
            self._mask = m
        return self._mask

    @torch.no_grad()
    def prefix(self, images, lang_ids, state):
        """images [B, n_cam, 3, H, W] in [0,1]; lang_ids [B, n_lang]; state [B, action_pad] → per-layer (K, V)."""
        c = self.c
        B = images.shape[0]
        dt = torch.bfloat16 if self.on_cuda else torch.float32
        it = self.vision.forward(images.reshape(B * c.n_cam, 3, c.image, c.image)).reshape(B, c.n_cam * c.tokens_per_image, c.hidden)
        lt = self.embed.forward(lang_ids) * math.sqrt(c.hidden)
        stt = self.state_proj.forward(state.to(dt) if self.on_cuda else state)[:, None]
        x = torch.cat([it.to(dt), lt.to(dt), stt.to(dt)], 1).contiguous()
        kv = []
        mask = self.prefix_mask(x.device)
        for blk in self.lm:
            x = blk.forward(x, bias=mask)
            kv.append((blk.attn.last_k.contiguous(), blk.attn.last_v.contiguous()))
            blk.release_buffers()
        return kv

    def suffix_embed(self, x_t, t):
        c = self.c
        B = x_t.shape[0]
        dt = torch.bfloat16 if self.on_cuda else torch.float32
        a = self.action_in.forward(x_t.to(dt)).to(dt)                                   # [B, chunk, W]
        te = nn.sincos_embed(t, c.expert_width).to(dt)[:, None].expand(B, c.chunk, c.expert_width)
        h = self.time_in.forward(torch.cat([a, te], -1).contiguous())
        return self.time_out.forward(h).to(dt)

    def denoise(self, kv, x_t, t):
        """Velocity prediction v(x_t, t) [B, chunk, action_pad] (fp32)."""
        h = self.suffix_embed(x_t, t)
        P = self.c.prefix_len
        for lyr, (pk, pv) in zip(self.expert, kv):
            h = lyr.forward(h, pk, pv, P)
        return self.action_out.forward(self.expert_norm.forward(h)).float()

    def denoise_vjp(self, dv):
        dt = torch.bfloat16 if self.on_cuda else torch.float32
        w = dv.shape[-1]
        d = dv.to(dt)
        dh = self.expert_norm.vjp(self.action_out.vjp(d.contiguous()))
        for lyr in reversed(self.expert):
            dh = lyr.vjp(dh)
        dcat = self.time_in.vjp(self.time_out.vjp(dh))
        self.action_in.vjp(dcat[..., : self.c.expert_width].contiguous())
        assert w == self.c.action_pad

    @torch.no_grad()
    def sample_actions(self, images, lang_ids, state, steps=10, generator=None):
        c = self.c
        kv = self.prefix(images, lang_ids, state)
        B = images.shape[0]
        x = torch.randn(B, c.chunk, c.action_pad, device=images.device, generator=generator)
        dtm = -1.0 / steps
        for s in range(steps):
            t = torch.full((B,), 1.0 + s * dtm, device=images.device)
            x = x + dtm * self.denoise(kv, x, t)
        return x[..., : c.action_dim]


class VLATrainer:
    def __init__(self, cfg: VLAConfig = None, device="cuda", grad_sync=None):
        self.cfg = cfg = cfg or VLAConfig()
        self.device = torch.device(device)
        self.model = VLAModel(cfg).to(self.device)
        for n, p in self.model.named_params():
            if n.startswith(("vision_model.", "text_model.")):
                p.frozen = True
        self.opt = nn.AdamW(self.model.trainable(), lr=cfg.lr, weight_decay=0.0)
        self.grad_sync = grad_sync
        if grad_sync is not None:
            grad_sync.attach(self.opt)
        self.loss_acc = torch.zeros(1, device=self.device)
        self.gen = torch.Generator(device=self.device).manual_seed(cfg.seed + 3)
        self.mse = nn.MSELoss()
        self._graphed = None

    def step(self, images, lang_ids, state, actions):
        """One optimisation step replayed from a CUDA graph (captured on the third call; shapes must stay fixed)."""
        if self._graphed is None:
            from ..utils.graphs import GraphedStep
            self._graphed = GraphedStep(self.train_step, [images, lang_ids, state, actions], generators=[self.gen])
        return self._graphed(images, lang_ids, state, actions)

    def train_step(self, images, lang_ids, state, actions):
        """images [B, n_cam, 3, H, W] in [0,1], lang_ids [B, n_lang] int64, state [B, action_dim], actions [B, chunk, action_dim]."""
        c, dev = self.cfg, self.device
        B = images.shape[0]
        st = torch.zeros(B, c.action_pad, device=dev)
        st[:, : state.shape[1]] = state
        act = torch.zeros(B, c.chunk, c.action_pad, device=dev)
        act[..., : c.action_dim] = actions
        kv = self.model.prefix(images, lang_ids, st)
        noise = torch.randn(act.shape, device=dev, generator=self.gen)
        u = torch.rand(B, device=dev, generator=self.gen)
        t = u.pow(1.0 / 1.5) * 0.999 + 0.001
        x_t = t[:, None, None] * noise + (1 - t[:, None, None]) * act
        target = noise - act
        v = self.model.denoise(kv, x_t, t)
        dv = self.mse(v, target, self.loss_acc, n_real=c.action_dim)
        self.model.denoise_vjp(dv)
        if self.grad_sync is not None:
            self.grad_sync.reduce_and_step(self.opt)
        else:
            self.opt.step(zero_grad=True)
        return self.loss_acc
