"""Dreamer 4: block-causal dynamics over a per-frame token grid, shortcut-forcing loss, MAE tokenizer, agent heads,
imagination RL losses and the few-step ODE sampler.

Everything is written against ``noeira_b200.nn`` modules with explicit backward passes (no tape), so the same code runs
on the CPU oracle path and on the GPU kernels (flash attention with ``Q_LEN != KV_LEN`` batches, fused GEMM epilogues).

  SpaceTimeBlock     pre-RMSNorm residual sublayers: space attention inside a frame (batch = B·T, S tokens), causal time
                     attention across frames per token position (batch = B·S, T tokens), SwiGLU FFN
                     (noeira/deep_agents/dreamer4/blocks.mojo:43-101)
  Dreamer4Dynamics   per-frame grid ``[action | signal | step | spatial×NSP | register×NREG | agent]`` with learned
                     ``action_base``, ``signal_table``, ``step_table``, ``register``, ``agent_base``; predicts the clean
                     latents (x-prediction) from the corrupted ones (dynamics.mojo:98-314)
  shortcut_forcing_loss   empirical rows: w(σ)·MSE(ẑ, z1); self rows: bootstrap target from two half steps, loss
                     w(σ)(1−σ)²·MSE((ẑ − z̃)/(1−σ), v̄); emits dL/dẑ (shortcut_loss.mojo:215-435)
  sample_one_timestep     K Euler steps of the shortcut model on the last frame given clean context (ode_sampler.mojo:41)
  policy / reward / value / continue heads   Linear → SiLU → Linear, multi-token-prediction outputs (heads.mojo)
  lambda_returns, value_td_loss, pmpo_policy_loss, continue_bce   imagination RL losses with their gradients
                     (imag_rl_loss.mojo:61-344)
  Dreamer4Tokenizer  masked-autoencoder tokenizer: patches → encoder → tanh bottleneck → decoder with learned patch
                     queries → sigmoid pixels (tokenizer.mojo:32, blocks.mojo:149-171); temporal_patchify / unpatchify
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Optional

import torch

from .. import nn
from ..nn.losses import symexp, symlog, two_hot
from ..nn.module import Module
from ..nn.transformer import RMSNorm, SelfAttention, SwiGLUFFN

UNIMIX = 0.01


# ------------------------------------------------------------------------------------------ blocks
class SpaceTimeBlock(Module):
    def __init__(self, dim: int, heads: int, ff: int):
        super().__init__()
        self.n1 = self.add_child("0.0", RMSNorm(dim))
        self.space = self.add_child("0.1", SelfAttention(dim, heads, bias=False))
        self.n2 = self.add_child("1.0", RMSNorm(dim))
        self.time = self.add_child("1.1", SelfAttention(dim, heads, mask="causal", bias=False))
        self.n3 = self.add_child("2.0", RMSNorm(dim))
        self.ffn = self.add_child("2.1", SwiGLUFFN(dim, ff))

    def forward(self, x):
        """x [B, T, S, D]"""
        B, T, S, D = x.shape
        self._shape = x.shape
        x = x + self.space.forward(self.n1.forward(x.reshape(B * T, S, D))).reshape(B, T, S, D)
        xt = x.permute(0, 2, 1, 3).reshape(B * S, T, D).contiguous()
        x = x + self.time.forward(self.n2.forward(xt)).reshape(B, S, T, D).permute(0, 2, 1, 3)
        return x + self.ffn.forward(self.n3.forward(x.reshape(B * T * S, D))).reshape(B, T, S, D)

    def vjp(self, dy):
        B, T, S, D = self._shape
        dx = dy + self.n3.vjp(self.ffn.vjp(dy.reshape(B * T * S, D).contiguous())).reshape(B, T, S, D)
        dt_ = dx.permute(0, 2, 1, 3).reshape(B * S, T, D).contiguous()
        dx = dx + self.n2.vjp(self.time.vjp(dt_)).reshape(B, S, T, D).permute(0, 2, 1, 3)
        return dx + self.n1.vjp(self.space.vjp(dx.reshape(B * T, S, D).contiguous())).reshape(B, T, S, D)


@dataclass
class Dreamer4Config:
    nsp: int = 16          # spatial latent tokens per frame
    dsp: int = 8           # channels per latent token
    dim: int = 64
    heads: int = 4
    ff: int = 128
    depth: int = 2
    nreg: int = 2
    kmax: int = 8          # finest signal grid (σ index 0 … kmax-1); step index e means d = 1/2^e
    adim: int = 0          # action components per frame (0 = unconditional)
    seed: int = 0

    @property
    def emax(self):
        return int(math.log2(self.kmax))

    @property
    def tokens(self):
        return 3 + self.nsp + self.nreg + 1


class Dreamer4Dynamics(Module):
    """x-prediction dynamics: ``forward(z̃ [B·T, NSP·DSP]) → ẑ`` with the frame's signal / step indices (and action)
    set beforehand through ``set_indices`` / ``set_actions`` — the ``ShortcutDynamics`` trait of the reference."""

    def __init__(self, cfg: Dreamer4Config, T: int):
        super().__init__()
        self.cfg, self.T = cfg, T
        nn.manual_seed(cfg.seed)
        D = cfg.dim
        self.inp = self.add_child("in_proj", nn.Linear(cfg.dsp, D))
        self.action_base = self.add_param("action_base", (1, D), decay=False, init=nn.Normal(0, 0.02))
        self.act_proj = self.add_child("action_proj", nn.Linear(max(cfg.adim, 1), D, bias=False)) if cfg.adim else None
        self.signal_table = self.add_param("signal_table", (cfg.kmax, D), decay=False, init=nn.Normal(0, 0.02))
        self.step_table = self.add_param("step_table", (cfg.emax + 1, D), decay=False, init=nn.Normal(0, 0.02))
        self.register = self.add_param("register", (cfg.nreg, D), decay=False, init=nn.Normal(0, 0.02))
        self.agent_base = self.add_param("agent_base", (1, D), decay=False, init=nn.Normal(0, 0.02))
        self.blocks = [self.add_child(f"blocks.{i}", SpaceTimeBlock(D, cfg.heads, cfg.ff)) for i in range(cfg.depth)]
        self.norm = self.add_child("out_norm", RMSNorm(D))
        self.out = self.add_child("out_proj", nn.Linear(D, cfg.dsp))
        self._sig = self._stp = self._act = None

    # ---- conditioning (per frame row)
    def set_indices(self, sigma_idx, step_idx):
        self._sig, self._stp = sigma_idx.long(), step_idx.long()

    def set_actions(self, actions, mask=None):
        self._act = None if actions is None else (actions if mask is None else actions * mask)

    def _w(self, p):
        return p.data

    def forward(self, z):
        c = self.cfg
        BF = z.shape[0]
        B = BF // self.T
        D = c.dim
        dev, dt = z.device, z.dtype
        sp = self.inp.forward(z.reshape(BF * c.nsp, c.dsp)).reshape(BF, c.nsp, D).to(dt)
        a = self._w(self.action_base).to(dt).expand(BF, 1, D)
        if self.act_proj is not None and self._act is not None:
            a = a + self.act_proj.forward(self._act.to(dt))[:, None].to(dt)
        sig = self._w(self.signal_table).to(dt)[self._sig][:, None]
        stp = self._w(self.step_table).to(dt)[self._stp][:, None]
        reg = self._w(self.register).to(dt)[None].expand(BF, c.nreg, D)
        ag = self._w(self.agent_base).to(dt).expand(BF, 1, D)
        x = torch.cat([a, sig, stp, sp, reg, ag], 1).reshape(B, self.T, c.tokens, D)
        for b in self.blocks:
            x = b.forward(x)
        self._agent_out = x[:, :, -1]
        h = self.norm.forward(x[:, :, 3: 3 + c.nsp].reshape(BF * c.nsp, D).contiguous())
        return self.out.forward(h).reshape(BF, c.nsp * c.dsp).to(dt)

    def agent_out(self):
        """Task-output embeddings h_t [B, T, D] read by the policy / reward / value heads."""
        return self._agent_out

    def vjp(self, dzhat, dagent=None):
        c = self.cfg
        BF = dzhat.shape[0]
        B, D = BF // self.T, c.dim
        dh = self.norm.vjp(self.out.vjp(dzhat.reshape(BF * c.nsp, c.dsp).contiguous()))
        dx = torch.zeros(B, self.T, c.tokens, D, dtype=dh.dtype, device=dh.device)
        dx[:, :, 3: 3 + c.nsp] = dh.reshape(B, self.T, c.nsp, D)
        if dagent is not None:
            dx[:, :, -1] += dagent.to(dx.dtype)
        for b in reversed(self.blocks):
            dx = b.vjp(dx)
        dx = dx.reshape(BF, c.tokens, D).float()
        self.action_base.grad.add_(dx[:, 0].sum(0, keepdim=True))
        if self.act_proj is not None and self._act is not None:
            self.act_proj.vjp(dx[:, 0].contiguous())
        self.signal_table.grad.index_add_(0, self._sig, dx[:, 1])
        self.step_table.grad.index_add_(0, self._stp, dx[:, 2])
        self.register.grad.add_(dx[:, 3 + c.nsp: 3 + c.nsp + c.nreg].sum(0))
        self.agent_base.grad.add_(dx[:, -1].sum(0, keepdim=True))
        self.inp.vjp(dx[:, 3: 3 + c.nsp].reshape(BF * c.nsp, D).contiguous())
        return None


# ------------------------------------------------------------------------------------------ shortcut forcing
def shortcut_forcing_loss(dyn, z1, z0, sigma, sigma_idx, step_idx, T: int, b_self: int, kmax: int, do_boot: bool = True,
                          actions=None, act_mask=None):
    """z1 / z0 [B·T, ND] clean latents / noise, sigma [B·T] signal level in [0, 1), sigma_idx / step_idx [B·T] integer
    indices; the LAST ``b_self`` sequences are self (bootstrap) rows.  Returns (loss, dL/dẑ [B·T, ND], ẑ).  The main
    forward runs last, so the module's caches serve ``dyn.vjp(grad)``."""
    BF, ND = z1.shape
    B = BF // T
    b_emp = B - b_self
    BS, S0 = b_self * T, (B - b_self) * T
    s = sigma[:, None]
    ztil = (1 - s) * z0 + s * z1
    zts = ztil[S0:]
    vbar = None
    if do_boot and b_self > 0:
        stp = step_idx[S0:].long()
        dh = 0.5 / (2.0 ** stp.double())
        sig_self = sigma[S0:].double()
        sig_plus = sig_self + dh
        step_half = stp + 1
        sidx = sigma_idx[S0:].long()
        sidx_plus = sidx + (kmax * dh).long()
        with torch.no_grad():
            # the two half-step passes run on the self sequences only (a sub-batch of whole sequences)
            dyn.set_actions(None if actions is None else actions[S0:], act_mask)
            dyn.set_indices(sidx, step_half)
            zh1 = dyn.forward(zts)
            bp = (zh1 - zts) / (1 - sig_self).clamp_min(1e-6)[:, None].to(zts.dtype)
            zprime = zts + bp * dh[:, None].to(zts.dtype)
            dyn.set_indices(sidx_plus.clamp_max(kmax - 1), step_half)
            zh2 = dyn.forward(zprime)
            bpp = (zh2 - zprime) / (1 - sig_plus).clamp_min(1e-6)[:, None].to(zts.dtype)
            vbar = (bp + bpp) / 2
    dyn.set_actions(actions, act_mask)
    dyn.set_indices(sigma_idx, step_idx)
    zhat = dyn.forward(ztil)
    pref = 1.0 / BF
    grad = torch.zeros_like(zhat)
    w = 0.9 * sigma + 0.1
    loss_emp = zhat.new_zeros(())
    if b_emp > 0:
        diff = zhat[:S0] - z1[:S0]
        loss_emp = (w[:S0] * diff.pow(2).mean(1)).sum() / (b_emp * T)
        grad[:S0] = pref * w[:S0, None] * (2.0 / ND) * diff
    loss_self = zhat.new_zeros(())
    if vbar is not None:
        sv = sigma[S0:]
        om = 1 - sv
        den = om.clamp_min(1e-6)
        d = (zhat[S0:] - zts) / den[:, None] - vbar
        loss_self = (w[S0:] * om * om * d.pow(2).mean(1)).sum() / BS
        grad[S0:] = pref * (w[S0:] * om * om / den)[:, None] * (2.0 / ND) * d
    loss = (loss_emp * b_emp + loss_self * b_self) / B
    return loss, grad, zhat


def sample_one_timestep(dyn, context, z_init, T: int, kmax: int, K: int, actions=None):
    """``context [B·(T−1), ND]`` clean frames, ``z_init [B, ND]`` noise → the next frame after K Euler steps of the
    shortcut model (step size 1/K: step index log2 K; context frames run at the finest level)."""
    B, ND = z_init.shape
    emax, e, scale = int(math.log2(kmax)), int(math.log2(K)), kmax // K
    packed = torch.zeros(B, T, ND, dtype=z_init.dtype, device=z_init.device)
    packed[:, : T - 1] = context.reshape(B, T - 1, ND)
    step_idx = torch.full((B, T), emax, dtype=torch.long, device=z_init.device)
    step_idx[:, -1] = e
    sig_idx = torch.full((B, T), kmax - 1, dtype=torch.long, device=z_init.device)
    z = z_init.clone()
    dyn.set_actions(actions)
    with torch.no_grad():
        for i in range(K):
            tau = i / K
            sig_idx[:, -1] = i * scale
            packed[:, -1] = z
            dyn.set_indices(sig_idx.reshape(-1), step_idx.reshape(-1))
            x1 = dyn.forward(packed.reshape(B * T, ND)).reshape(B, T, ND)[:, -1]
            z = z + (x1 - z) / max(1e-4, 1 - tau) / K
    return z


# ------------------------------------------------------------------------------------------ heads and RL losses
def policy_head(d_in, hid, nact, nmtp=1):
    return nn.Sequential(nn.Linear(d_in, hid, act="silu"), nn.Linear(hid, nmtp * nact))


def reward_head(d_in, hid, nbins, nmtp=1):
    return nn.Sequential(nn.Linear(d_in, hid, act="silu"), nn.Linear(hid, nmtp * nbins))


def value_head(d_in, hid, nbins):
    return nn.Sequential(nn.Linear(d_in, hid, act="silu"), nn.Linear(hid, nbins))


def continue_head(d_in, hid):
    return nn.Sequential(nn.Linear(d_in, hid, act="silu"), nn.Linear(hid, 1))


def lambda_returns(rew, val, con, lam: float):
    """rew / val / con [B, H] (reward and discount·(1−done) ARRIVING at state t) → R^λ [B, H−1]."""
    B, H = rew.shape
    out = torch.zeros(B, H - 1, dtype=rew.dtype, device=rew.device)
    nxt = val[:, H - 1]
    for t in range(H - 2, -1, -1):
        live = con[:, t + 1]
        nxt = rew[:, t + 1] + (1 - lam) * live * val[:, t + 1] + live * lam * nxt
        out[:, t] = nxt
    return out


def value_td_loss(vlogits, returns, bins):
    """Two-hot cross entropy of value logits [B, H, BINS] against sg(λ-return) [B, H−1] (symlog space); returns
    (loss, dL/dlogits)."""
    B, H, NB = vlogits.shape
    lg = vlogits[:, : H - 1].reshape(-1, NB).float()
    tgt = two_hot(symlog(returns.reshape(-1).float()), bins)
    logp = torch.log_softmax(lg, -1)
    n = lg.shape[0]
    loss = -(tgt * logp).sum(-1).mean()
    g = torch.zeros_like(vlogits, dtype=torch.float32)
    g[:, : H - 1] = ((logp.exp() - tgt) / n).reshape(B, H - 1, NB)
    return loss, g


def _unimix_probs(logits):
    p = torch.softmax(logits.float(), -1)
    return (1 - UNIMIX) * p + UNIMIX / logits.shape[-1], p


def pmpo_policy_loss(plogits, prior_logits, actions, adv, alpha: float = 0.5, beta: float = 0.3):
    """PMPO: −(1−α)/|D⁺| Σ_{A≥0} log π(a) + α/|D⁻| Σ_{A<0} log π(a) + β/N Σ KL(π ‖ π_prior) over the H−1 imagined steps,
    categorical π with 1 % uniform mix.  plogits / prior_logits [B, H, NACT], actions [B, H] class ids, adv [B, H−1].
    Returns (loss, dL/dplogits)."""
    B, H, NA = plogits.shape
    lg = plogits[:, : H - 1].float()
    pm, sm = _unimix_probs(lg)
    qm, _ = _unimix_probs(prior_logits[:, : H - 1])
    a = actions[:, : H - 1].long()
    logp = torch.log(pm.gather(-1, a[..., None]).squeeze(-1))
    pos = adv >= 0
    n_pos, n_neg, N = int(pos.sum()), int((~pos).sum()), B * (H - 1)
    coef = torch.where(pos, -(1 - alpha) / max(n_pos, 1), alpha / max(n_neg, 1)).to(logp.dtype)
    kl = (pm * (torch.log(pm) - torch.log(qm))).sum(-1)
    loss = (coef * logp).sum() + beta / N * kl.sum()
    # gradient w.r.t. the mixed probabilities, then through mix and softmax
    onehot = torch.nn.functional.one_hot(a, NA).to(pm.dtype)
    dpm = coef[..., None] * onehot / pm + beta / N * (torch.log(pm) - torch.log(qm) + 1)
    dsm = (1 - UNIMIX) * dpm
    dlg = sm * (dsm - (dsm * sm).sum(-1, keepdim=True))
    g = torch.zeros_like(plogits, dtype=torch.float32)
    g[:, : H - 1] = dlg
    return loss, g


def continue_bce(clogit, cont_target):
    """Binary cross entropy of the continue logit against 1 − done; returns (loss, dL/dlogit)."""
    x, y = clogit.float().reshape(-1), cont_target.float().reshape(-1)
    loss = (torch.clamp(x, min=0) - x * y + torch.log1p(torch.exp(-x.abs()))).mean()
    return loss, ((torch.sigmoid(x) - y) / x.numel()).reshape(clogit.shape)


# ------------------------------------------------------------------------------------------ tokenizer
def temporal_patchify(frames, patch: int):
    """frames [B, T, C, H, W] → [B·T, (H/p)(W/p), C·p·p]"""
    B, T, C, H, W = frames.shape
    g, h = H // patch, W // patch
    x = frames.reshape(B * T, C, g, patch, h, patch).permute(0, 2, 4, 1, 3, 5)
    return x.reshape(B * T, g * h, C * patch * patch).contiguous()


def temporal_unpatchify(tokens, patch: int, C: int, H: int, W: int, T: int):
    BT = tokens.shape[0]
    g, h = H // patch, W // patch
    x = tokens.reshape(BT, g, h, C, patch, patch).permute(0, 3, 1, 4, 2, 5)
    return x.reshape(BT // T, T, C, H, W).contiguous()


def downscale_box(frames, factor: int):
    return torch.nn.functional.avg_pool2d(frames.reshape(-1, *frames.shape[-3:]), factor).reshape(*frames.shape[:-2],
                                                                                               frames.shape[-2] // factor,
                                                                                               frames.shape[-1] // factor)


class Dreamer4Tokenizer(Module):
    """Masked-autoencoder tokenizer over the patches of one frame: encoder blocks → ``NSP`` latent tokens through a
    learned-query read-out and a tanh bottleneck of ``DSP`` channels; decoder: up-projection, learned patch queries with
    sinusoidal positions, blocks, patch head, sigmoid.  ``forward(patches, mask)`` returns the reconstruction;
    ``vjp`` takes dL/drecon."""

    def __init__(self, n_patches: int, patch_dim: int, nsp: int, dsp: int, dim: int = 64, heads: int = 4, ff: int = 128,
                 depth: int = 2, seed: int = 0):
        super().__init__()
        nn.manual_seed(seed)
        self.np_, self.pd, self.nsp, self.dsp, self.dim = n_patches, patch_dim, nsp, dsp, dim
        self.embed = self.add_child("patch_embed", nn.Linear(patch_dim, dim))
        self.mask_token = self.add_param("mask_token", (1, dim), decay=False, init=nn.Normal(0, 0.02))
        self.lat_q = self.add_param("latent_queries", (nsp, dim), decay=False, init=nn.Normal(0, 0.02))
        self.enc = [self.add_child(f"encoder.{i}", nn.TransformerBlock(dim, heads, ff, norm="rms", ffn="swiglu", bias=False))
                    for i in range(depth)]
        self.down = self.add_child("down_proj", nn.Linear(dim, dsp, act="tanh"))
        self.up = self.add_child("up_proj", nn.Linear(dsp, dim, act="tanh"))
        self.patch_q = self.add_param("patch_queries", (n_patches, dim), decay=False, init=nn.Normal(0, 0.02))
        self.dec = [self.add_child(f"decoder.{i}", nn.TransformerBlock(dim, heads, ff, norm="rms", ffn="swiglu", bias=False))
                    for i in range(depth)]
        self.head = self.add_child("patch_head", nn.Linear(dim, patch_dim, act="sigmoid"))
        pos = torch.arange(n_patches + nsp, dtype=torch.float32)
        self.pos = nn.sincos_embed(pos / (n_patches + nsp), dim, min_period=1.0 / (n_patches + nsp), max_period=4.0) / math.sqrt(dim)

    def encode(self, patches, mask=None):
        """patches [N, NP, PD]; mask [N, NP] with 1 = hidden from the encoder.  Returns latents [N, NSP·DSP]."""
        N, dt = patches.shape[0], patches.dtype
        x = self.embed.forward(patches.reshape(N * self.np_, self.pd)).reshape(N, self.np_, self.dim).to(dt)
        self._mask = mask
        if mask is not None:
            m = mask[..., None].to(dt)
            x = x * (1 - m) + self.mask_token.data.to(dt)[None] * m
        x = torch.cat([x, self.lat_q.data.to(dt)[None].expand(N, self.nsp, self.dim)], 1) + self.pos.to(patches.device, dt)[None]
        for b in self.enc:
            x = b.forward(x)
        self._n = N
        z = self.down.forward(x[:, self.np_:].reshape(N * self.nsp, self.dim).contiguous())
        return z.reshape(N, self.nsp * self.dsp).to(dt)

    def decode(self, z):
        N, dt = z.shape[0], z.dtype
        u = self.up.forward(z.reshape(N * self.nsp, self.dsp)).reshape(N, self.nsp, self.dim).to(dt)
        x = torch.cat([self.patch_q.data.to(dt)[None].expand(N, self.np_, self.dim), u], 1) + self.pos.to(z.device, dt)[None]
        for b in self.dec:
            x = b.forward(x)
        return self.head.forward(x[:, : self.np_].reshape(N * self.np_, self.dim).contiguous()).reshape(N, self.np_, self.pd).to(dt)

    def forward(self, patches, mask=None):
        return self.decode(self.encode(patches, mask))

    def vjp(self, drecon):
        N = self._n
        dx = torch.zeros(N, self.np_ + self.nsp, self.dim, dtype=drecon.dtype, device=drecon.device)
        dx[:, : self.np_] = self.head.vjp(drecon.reshape(N * self.np_, self.pd).contiguous()).reshape(N, self.np_, self.dim)
        for b in reversed(self.dec):
            dx = b.vjp(dx)
        self.patch_q.grad.add_(dx[:, : self.np_].float().sum(0))
        dz = self.up.vjp(dx[:, self.np_:].reshape(N * self.nsp, self.dim).contiguous())
        return self.encode_vjp(dz.reshape(N, self.nsp * self.dsp))

    def encode_vjp(self, dz):
        N = self._n
        dx = torch.zeros(N, self.np_ + self.nsp, self.dim, dtype=dz.dtype, device=dz.device)
        dx[:, self.np_:] = self.down.vjp(dz.reshape(N * self.nsp, self.dsp).contiguous()).reshape(N, self.nsp, self.dim)
        for b in reversed(self.enc):
            dx = b.vjp(dx)
        self.lat_q.grad.add_(dx[:, self.np_:].float().sum(0))
        dp = dx[:, : self.np_]
        if self._mask is not None:
            m = self._mask[..., None].to(dp.dtype)
            self.mask_token.grad.add_((dp * m).float().sum((0, 1))[None])
            dp = dp * (1 - m)
        self.embed.vjp(dp.reshape(N * self.np_, self.dim).contiguous())
        return None


def mae_mask(n: int, n_patches: int, p_min: float, p_max: float, gen: Optional[torch.Generator] = None, device="cpu"):
    """Per-sample masking ratio U(p_min, p_max); returns [n, n_patches] with 1 = masked."""
    ratio = p_min + (p_max - p_min) * torch.rand(n, 1, generator=gen, device=device)
    return (torch.rand(n, n_patches, generator=gen, device=device) < ratio).float()


# ------------------------------------------------------------------------------------------ agent facade
class Dreamer4Agent:
    """The three training phases over one dynamics model and its heads
    (noeira/deep_agents/dreamer4/agent.mojo:79-169, 716-1099):

      ``bc_train_step``    video prediction (shortcut forcing on the latents) + behaviour cloning of the policy head on the
                           agent-token outputs, one backward through the dynamics carrying both gradients
      ``acwm_train_step``  action-conditioned world model + reward / continue heads
      ``imag_train_step``  imagination RL with the dynamics frozen: roll the model forward from context frames with actions
                           of the policy head (one shortcut sample of ``K`` Euler steps per frame), λ-returns, two-hot value
                           TD loss, PMPO policy loss with a KL pull to the frozen behavioural prior

    Latents ``z [B, T, NSP·DSP]`` come from the tokenizer; actions are discrete (one-hot conditioning, ``cfg.adim`` =
    number of actions)."""

    def __init__(self, cfg: Dreamer4Config, T: int, n_actions: int, n_bins: int = 41, head_hidden: int = 64, lr: float = 1e-3,
                 gamma: float = 0.97, lam: float = 0.95, device="cpu"):
        assert cfg.adim == n_actions, "discrete actions condition the dynamics as one-hot vectors: cfg.adim = n_actions"
        self.cfg, self.T, self.nact, self.gamma, self.lam = cfg, T, n_actions, gamma, lam
        self.device = torch.device(device)
        self.dyn = Dreamer4Dynamics(cfg, T).to(self.device)
        D = cfg.dim
        nn.manual_seed(cfg.seed + 7)
        self.ph, self.ph_prior = policy_head(D, head_hidden, n_actions).to(self.device), policy_head(D, head_hidden, n_actions).to(self.device)
        self.rh, self.vh, self.ch = reward_head(D, head_hidden, n_bins).to(self.device), value_head(D, head_hidden, n_bins).to(self.device), \
            continue_head(D, head_hidden).to(self.device)
        self.ph_prior.copy_from(self.ph)
        self.bins = torch.linspace(-10.0, 10.0, n_bins, device=self.device)
        # one optimizer per group that a phase may freeze: a zero gradient alone would still move parameters through
        # Adam's running moments
        self.wm_opt = nn.Adam(list(self.dyn.named_params("dyn.")) + list(self.rh.named_params("rh.")) + list(self.ch.named_params("ch.")), lr=lr)
        self.ph_opt = nn.Adam(self.ph.named_params("ph."), lr=lr)
        self.vh_opt = nn.Adam(self.vh.named_params("vh."), lr=lr)
        for o in (self.wm_opt, self.ph_opt, self.vh_opt):
            o.max_grad_norm = 10.0
        self.gen = torch.Generator(device=self.device).manual_seed(cfg.seed + 11)

    def named_params(self):
        yield from self.dyn.named_params("dyn.")
        for k, m in (("ph", self.ph), ("rh", self.rh), ("vh", self.vh), ("ch", self.ch)):
            yield from m.named_params(k + ".")

    # ---- shared: noise levels of a shortcut-forcing batch
    def _levels(self, B, b_self):
        """Signal level and step index per frame row: the first ``B − b_self`` sequences train at the finest step against
        the data (flow-matching rows), the last ``b_self`` at a coarser step d = 1 / 2^e, e < emax, against two half steps."""
        c, T = self.cfg, self.T
        n, ns = B * T, b_self * T
        step = torch.full((n,), c.emax, device=self.device, dtype=torch.long)
        if ns:
            step[n - ns:] = torch.randint(0, max(c.emax, 1), (ns,), device=self.device, generator=self.gen)
        grid = 2 ** step
        k = (torch.rand(n, device=self.device, generator=self.gen) * grid).long().clamp(max=c.kmax - 1)
        k = torch.minimum(k, grid - 1)
        sigma_idx = k * (c.kmax // grid)
        return sigma_idx.float() / c.kmax, sigma_idx, step

    def _one_hot(self, a):
        return torch.nn.functional.one_hot(a.long().reshape(-1), self.nact).float()

    def _wm_pass(self, z, actions):
        B, T, ND = z.shape
        z1 = z.reshape(B * T, ND)
        z0 = torch.randn(z1.shape, device=self.device, generator=self.gen)
        b_self = B // 4 if self.cfg.emax > 0 else 0
        sigma, sidx, stp = self._levels(B, b_self)
        return shortcut_forcing_loss(self.dyn, z1, z0, sigma, sidx, stp, T, b_self, self.cfg.kmax, do_boot=b_self > 0,
                                     actions=None if actions is None else self._one_hot(actions))

    @staticmethod
    def _finish(*opts):
        for o in opts:
            if o.max_grad_norm > 0:
                o.clip()
            o.step(zero_grad=True)

    def bc_train_step(self, z, actions):
        """z [B, T, ND], actions [B, T] (the action taken at frame t): video prediction + BC."""
        B, T, _ = z.shape
        loss, grad, _ = self._wm_pass(z, None)
        h = self.dyn.agent_out().reshape(B * T, -1)
        logits = self.ph.forward(h).float()
        logp = torch.log_softmax(logits, -1)
        onehot = self._one_hot(actions)
        bc = -(onehot * logp).sum(-1).mean()
        dh = self.ph.vjp((logp.exp() - onehot) / (B * T))
        self.dyn.vjp(grad, dh.reshape(B, T, -1))
        self._finish(self.wm_opt, self.ph_opt)
        return dict(wm_loss=float(loss), bc_loss=float(bc))

    def acwm_train_step(self, z, actions, rewards, cont):
        """Action-conditioned world model + reward and continue heads (rewards / cont [B, T] arriving at frame t)."""
        B, T, _ = z.shape
        loss, grad, _ = self._wm_pass(z, actions)
        h = self.dyn.agent_out().reshape(B * T, -1)
        rl, drl = two_hot_ce(self.rh.forward(h).float(), rewards.reshape(-1), self.bins)
        cl, dcl = continue_bce(self.ch.forward(h).float(), cont.reshape(-1, 1))
        dh = self.rh.vjp(drl) + self.ch.vjp(dcl)
        self.dyn.vjp(grad, dh.reshape(B, T, -1))
        self._finish(self.wm_opt)
        return dict(wm_loss=float(loss), reward_loss=float(rl), cont_loss=float(cl))

    @torch.no_grad()
    def _features(self, window, acts):
        """Agent-token outputs of a window of clean frames ``[B, T, ND]`` (finest signal level, one-step index)."""
        c, (B, T, ND) = self.cfg, window.shape
        self.dyn.set_actions(acts.reshape(B * T, -1))
        self.dyn.set_indices(torch.full((B * T,), c.kmax - 1, device=self.device), torch.full((B * T,), c.emax, device=self.device))
        self.dyn.forward(window.reshape(B * T, ND))
        return self.dyn.agent_out()[:, -1]

    def imag_train_step(self, context, context_actions, horizon: int = 6, K: int = 2, alpha: float = 0.5, beta: float = 0.3):
        """context [B, T, ND] real latents, context_actions [B, T]: imagine ``horizon`` frames, train value and policy heads."""
        c, (B, T, ND) = self.cfg, context.shape
        win, acts = context.clone(), self._one_hot(context_actions).reshape(B, T, -1)
        feats, actions = [], []
        for _ in range(horizon):
            h = self._features(win, acts)                                         # state of the newest frame
            with torch.no_grad():
                a = torch.multinomial(_unimix_probs(self.ph.forward(h).float())[0], 1, generator=self.gen)[:, 0]
            feats.append(h), actions.append(a)
            a_win = torch.cat([acts[:, 1:], self._one_hot(a)[:, None]], 1)        # the new action conditions the next frame
            z_next = sample_one_timestep(self.dyn, win[:, 1:].reshape(B * (T - 1), ND), torch.randn(B, ND, device=self.device, generator=self.gen),
                                         T, c.kmax, K, actions=a_win.reshape(B * T, -1))
            win, acts = torch.cat([win[:, 1:], z_next[:, None]], 1), a_win
        feats.append(self._features(win, acts))
        F_ = torch.stack(feats, 1).detach()                                       # [B, H+1, D]
        A_ = torch.stack(actions + [actions[-1]], 1)
        H1 = horizon + 1
        flat = F_.reshape(B * H1, -1)
        with torch.no_grad():
            rew = symexp((torch.softmax(self.rh.forward(flat).float(), -1) * self.bins).sum(-1)).reshape(B, H1)
            con = self.gamma * torch.sigmoid(self.ch.forward(flat).float()).reshape(B, H1)
        vlogits = self.vh.forward(flat).float().reshape(B, H1, -1)
        val = symexp((torch.softmax(vlogits, -1) * self.bins).sum(-1)).detach()
        ret = lambda_returns(rew, val, con, self.lam)
        vloss, dv = value_td_loss(vlogits, ret, self.bins)
        self.vh.vjp(dv.reshape(B * H1, -1))
        plogits = self.ph.forward(flat).float().reshape(B, H1, -1)
        with torch.no_grad():
            prior = self.ph_prior.forward(flat).float().reshape(B, H1, -1)
        ploss, dp = pmpo_policy_loss(plogits, prior, A_, ret - val[:, :-1], alpha, beta)
        self.ph.vjp(dp.reshape(B * H1, -1))
        self._finish(self.ph_opt, self.vh_opt)                                    # the world model's optimizer does not step
        return dict(value_loss=float(vloss), policy_loss=float(ploss), imag_return=float(ret.mean()), imag_reward=float(rew[:, 1:].mean()))


def two_hot_ce(logits, target, bins):
    """Cross entropy against the two-hot encoding of symlog(target); returns (loss, dL/dlogits)."""
    tgt = two_hot(symlog(target.float()), bins)
    logp = torch.log_softmax(logits.float(), -1)
    return -(tgt * logp).sum(-1).mean(), (logp.exp() - tgt) / logits.shape[0]
