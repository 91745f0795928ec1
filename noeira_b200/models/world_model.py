"""Dreamer-style world-model dynamics transformer, tensor parallel with sequence-parallel activations.

Architecture (BASELINE configuration): 24 pre-RMSNorm blocks, d = 2048, 16 query heads / 4 KV heads (GQA),
head_dim 128, SwiGLU FF 5632, block-causal attention over 64 frames × (256 latent tokens + 1 action token):
full attention inside a frame, causal across frames — the reference factorises this as space attention +
causal time attention (noeira/deep_agents/dreamer4/blocks.mojo:1-101); here it is ONE block-causal flash
kernel.  Latents ~N(0,1)^32 are projected in, each frame carries one 6-dim action token, the loss is flow
matching (velocity prediction) on the latent tokens, AdamW lr 3e-4.

Parallel layout over P ranks (P = 1 runs the same code on one GPU):
  * rows (= batch·tokens) of every tensor outside attention / FFN are sharded across ranks (rank r holds rows
    [r·Ms, (r+1)·Ms)); norms, residuals, projections in/out and the loss run on the shard;
  * QKV and FFN-up are column parallel: all-gather → GEMM in one kernel (rows pulled from the peers' shards);
  * attention is head parallel: each rank owns Hq/P query heads and one KV head (KV heads are replicated across
    Hq/Hkv-sized... P/Hkv ranks; their gradients are summed over that replica group);
  * attention-out and FFN-down are row parallel: GEMM → reduce-scatter in one kernel, residual added in its
    epilogue;
  * replicated parameters (norm gains, in/out projections, time MLP) get their gradients all-reduced by the
    fused all-reduce + AdamW kernel; sharded parameters use the local arena AdamW.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass

import torch
import torch.distributed as dist

from .. import nn, ops
from .._native import check, cuda_lib, ptr, stream_ptr
from ..nn.init import Normal, Zero
from ..nn.layers import colsum_into
from ..nn.param import Param
from ..ops.attention import flash_attention_backward, flash_attention_forward
from ..parallel.tp import TPLinearContext


@dataclass
class WorldModelConfig:
    layers: int = 24
    dim: int = 2048
    heads: int = 16
    kv_heads: int = 4
    head_dim: int = 128
    ff: int = 5632
    frames: int = 64
    tokens_per_frame: int = 256
    latent_dim: int = 32
    action_dim: int = 6
    lr: float = 3e-4
    weight_decay: float = 0.0
    seed: int = 0

    @property
    def frame_len(self):
        return self.tokens_per_frame + 1

    @property
    def seq_len(self):
        return self.frames * self.frame_len

    def padded_seq_len(self, multiple=128):
        return (self.seq_len + multiple - 1) // multiple * multiple

    def num_params(self):
        d, hd = self.dim, self.head_dim
        per = d * (self.heads + 2 * self.kv_heads) * hd + self.heads * hd * d + 3 * d * self.ff + 2 * d
        return self.layers * per + (self.latent_dim + self.action_dim + 2) * d * 2 + d * d


def _mk(name, shape, std, gen, decay=True, fill=None):
    p = Param(name, shape, decay=decay, device=gen.device)
    if fill is not None:
        p.set_(torch.full(shape, float(fill)))
    else:
        p.set_(torch.randn(shape, generator=gen, device=gen.device) * std)
    return p


class TPBlock:
    """One transformer block with the TP + SP layout described in the module docstring."""

    def __init__(self, idx, cfg: WorldModelConfig, world, rank, gen, device):
        d, hd = cfg.dim, cfg.head_dim
        self.cfg, self.world, self.rank = cfg, world, rank
        if cfg.heads % world:
            raise ValueError(f"{cfg.heads} query heads do not split over {world} ranks")
        if world > cfg.kv_heads and world % cfg.kv_heads:
            raise ValueError(f"{world} ranks must be a multiple of the {cfg.kv_heads} KV heads they replicate")
        if world <= cfg.kv_heads and cfg.kv_heads % world:
            raise ValueError(f"{cfg.kv_heads} KV heads do not split over {world} ranks")
        self.hq = cfg.heads // world
        self.hkv = max(cfg.kv_heads // world, 1)
        self.kv_rep = max(world // cfg.kv_heads, 1)       # ranks sharing one KV head
        if cfg.ff % world or (cfg.ff // world) % 8:
            raise ValueError(f"ff = {cfg.ff} must split over {world} ranks into multiples of 8 columns")
        self.ffl = cfg.ff // world
        n_qkv = (self.hq + 2 * self.hkv) * hd
        pre = f"blocks.{idx}."
        # sharded parameters: every rank draws the FULL matrices from the same stream and keeps its slice, so the
        # model is identical for any P
        rn = lambda *shape: torch.randn(*shape, generator=gen, device=gen.device)
        wq = rn(d, cfg.heads * hd) * (1 / math.sqrt(d))
        wk = rn(d, cfg.kv_heads * hd) * (1 / math.sqrt(d))
        wv = rn(d, cfg.kv_heads * hd) * (1 / math.sqrt(d))
        wo = rn(cfg.heads * hd, d) * (1 / math.sqrt(cfg.heads * hd) / math.sqrt(2 * cfg.layers))
        wg = rn(d, cfg.ff) * (1 / math.sqrt(d))
        wu = rn(d, cfg.ff) * (1 / math.sqrt(d))
        wd = rn(cfg.ff, d) * (1 / math.sqrt(cfg.ff) / math.sqrt(2 * cfg.layers))
        q0 = rank * self.hq * hd
        kvh = (rank // self.kv_rep) * self.hkv * hd if world >= cfg.kv_heads else rank * self.hkv * hd
        dev = gen.device
        self.w_qkv = Param(pre + "attn.qkv.weight", (d, n_qkv), device=dev)
        self.w_qkv.set_(torch.cat([wq[:, q0:q0 + self.hq * hd], wk[:, kvh:kvh + self.hkv * hd], wv[:, kvh:kvh + self.hkv * hd]], 1))
        self.w_out = Param(pre + "attn.out.weight", (self.hq * hd, d), device=dev)
        self.w_out.set_(wo[q0:q0 + self.hq * hd])
        f0 = rank * self.ffl
        self.w_up = Param(pre + "ffn.0.weight", (d, 2 * self.ffl), device=dev)
        self.w_up.set_(torch.cat([wg[:, f0:f0 + self.ffl], wu[:, f0:f0 + self.ffl]], 1))
        self.w_down = Param(pre + "ffn.1.weight", (self.ffl, d), device=dev)
        self.w_down.set_(wd[f0:f0 + self.ffl])
        self.g1 = _mk(pre + "norm1.gamma", (d,), 0, gen, decay=False, fill=1.0)
        self.g2 = _mk(pre + "norm2.gamma", (d,), 0, gen, decay=False, fill=1.0)
        self.sharded = [self.w_qkv, self.w_out, self.w_up, self.w_down]
        self.replicated = [self.g1, self.g2]


class WorldModel:
    """Trainer-facing model object: ``loss = model.train_step(latents, actions)``."""

    def __init__(self, cfg: WorldModelConfig, batch: int, world: int = 1, rank: int = 0, device="cuda", group=None,
                 grad_sync=None):
        self.cfg, self.world, self.rank, self.group = cfg, world, rank, group
        self.device = torch.device(device)
        self.B = batch
        self.S = cfg.padded_seq_len(128)
        rows = batch * self.S
        if rows % (world * 128):
            raise ValueError(f"batch x padded sequence = {rows} rows must split into whole 128-row blocks on {world} ranks")
        self.ms = rows // world
        self.rows = rows
        d, hd = cfg.dim, cfg.head_dim
        # weights are drawn on the device (same seed → same full matrices on every rank, each keeps its slice)
        gen = torch.Generator(device=self.device).manual_seed(cfg.seed)
        nn.manual_seed(cfg.seed)
        self.in_lat = nn.Linear(cfg.latent_dim, d, bias=False, need_input_grad=False).to(self.device)
        self.in_act = nn.Linear(cfg.action_dim, d, bias=False, need_input_grad=False).to(self.device)
        self.t_lin = nn.Linear(d, d, act="silu", bias=False, need_input_grad=False).to(self.device)
        self.out_lin = nn.Linear(d, cfg.latent_dim, bias=False).to(self.device)
        self.out_g = _mk("out_norm.gamma", (d,), 0, gen, decay=False, fill=1.0)
        self.blocks = [TPBlock(i, cfg, world, rank, gen, self.device) for i in range(cfg.layers)]
        named_rep = (list(self.in_lat.named_params("in_latent.")) + list(self.in_act.named_params("in_action."))
                     + list(self.t_lin.named_params("time.")) + list(self.out_lin.named_params("out."))
                     + [(self.out_g.name, self.out_g)] + [(p.name, p) for b in self.blocks for p in b.replicated])
        rep = [p for _, p in named_rep]
        shd = [p for b in self.blocks for p in b.sharded]
        self.opt_rep = nn.AdamW(named_rep, lr=cfg.lr, weight_decay=cfg.weight_decay)
        self.opt_shd = nn.AdamW([(p.name, p) for p in shd], lr=cfg.lr, weight_decay=cfg.weight_decay)
        self.grad_sync = grad_sync
        if grad_sync is not None:
            grad_sync.attach(self.opt_rep)
            self.opt_rep.hyper[8] = 1.0  # gradients of replicated params are SUMMED over token shards
        b0 = self.blocks[0]
        mk = lambda k, n, kind, stage=True: TPLinearContext(world, rank, self.ms, k, n, kind, group, alloc_stage=stage)
        self.c_qkv = mk(d, (b0.hq + 2 * b0.hkv) * hd, "ag", False)
        self.c_out = mk(b0.hq * hd, d, "rs")
        self.c_up = mk(d, 2 * b0.ffl, "ag", False)
        self.c_down = mk(b0.ffl, d, "rs")
        # backward contexts
        self.cb_down = mk(d, b0.ffl, "ag")       # dY_shard → gather → · W_downᵀ
        self.cb_up = mk(2 * b0.ffl, d, "rs")     # dgu · W_upᵀ → reduce-scatter
        self.cb_out = mk(d, b0.hq * hd, "ag")
        self.cb_qkv = mk((b0.hq + 2 * b0.hkv) * hd, d, "rs")
        self.loss_acc = torch.zeros(1, device=self.device)
        self.lib = cuda_lib()
        self._ws = torch.empty(1 << 22, device=self.device)
        # positional table for the shard rows (sinusoidal over the position inside the sequence)
        pos = (torch.arange(self.ms, device=self.device) + rank * self.ms) % self.S
        self.pos = nn.sincos_embed(pos.float() / 64.0, d, min_period=1.0, max_period=float(self.S)).contiguous()
        # which shard rows are latent tokens / action tokens / padding
        fr, within = pos // cfg.frame_len, pos % cfg.frame_len
        self.is_lat = ((pos < cfg.seq_len) & (within > 0)).float()
        self.is_act = ((pos < cfg.seq_len) & (within == 0)).float()
        # ranks that replicate one KV head sum that head's weight gradients among themselves: one packed buffer, one
        # collective per step.  The group's communicator is created AND used once here, so that its set-up cost (which
        # differs from rank to rank) is not paid between two fused kernels of the first training step.
        self.kv_group, self._kv_pack = None, None
        if world > cfg.kv_heads:
            if not dist.is_initialized():
                raise RuntimeError("KV-head replica groups need an initialised process group")
            rep_n = world // cfg.kv_heads
            for g0 in range(0, world, rep_n):
                grp = dist.new_group(list(range(g0, g0 + rep_n)))
                if g0 <= rank < g0 + rep_n:
                    self.kv_group = grp
            kvw = 2 * b0.hkv * hd
            self._kv_pack = torch.zeros(cfg.layers, d, kvw, device=self.device)
            dist.all_reduce(self._kv_pack[0, :1], group=self.kv_group)
            torch.cuda.synchronize()
            dist.barrier(group=group)

    # ------------------------------------------------------------------ kernels
    def _norm_fwd(self, x, gamma, out):
        stats = torch.empty(x.shape[0], 2, device=x.device, dtype=torch.float32)
        check(self.lib.nb_norm_fwd(ptr(x), ctypes.c_int(x.stride(0)), ptr(gamma.storage), None, ptr(out), ctypes.c_int(out.stride(0)),
                                   ptr(stats), ctypes.c_int(x.shape[0]), ctypes.c_int(x.shape[1]), ctypes.c_float(1e-5),
                                   ctypes.c_int(1), stream_ptr()), "norm_fwd")
        return stats

    def _norm_bwd(self, x, dy, gamma, stats):
        dx = torch.empty_like(x)
        split = self.lib.nb_norm_split(ctypes.c_int(x.shape[0]))
        assert 2 * split * x.shape[1] <= self._ws.numel()
        check(self.lib.nb_norm_bwd(ptr(x), ctypes.c_int(x.stride(0)), ptr(dy), ctypes.c_int(dy.stride(0)), ptr(gamma.storage),
                                   ptr(stats), ptr(dx), ctypes.c_int(dx.stride(0)), ptr(gamma.grad_storage), None, ptr(self._ws),
                                   ctypes.c_int(x.shape[0]), ctypes.c_int(x.shape[1]), ctypes.c_int(1), ctypes.c_int(0),
                                   stream_ptr()), "norm_bwd")
        return dx

    def _swiglu(self, gu, H):
        h = torch.empty(gu.shape[0], H, device=gu.device, dtype=torch.bfloat16)
        check(self.lib.nb_swiglu_fwd(ptr(gu), ctypes.c_int(gu.stride(0)), ptr(h), ctypes.c_int(H), ctypes.c_int(gu.shape[0]),
                                     ctypes.c_int(H), stream_ptr()), "swiglu_fwd")
        return h

    def _swiglu_bwd(self, gu, dh, H):
        dgu = torch.empty_like(gu)
        check(self.lib.nb_swiglu_bwd(ptr(gu), ctypes.c_int(gu.stride(0)), ptr(dh), ctypes.c_int(dh.stride(0)), ptr(dgu),
                                     ctypes.c_int(gu.shape[0]), ctypes.c_int(H), stream_ptr()), "swiglu_bwd")
        return dgu

    # ------------------------------------------------------------------ block forward / backward
    def _block_fwd(self, blk: TPBlock, x):
        cfg, hd = self.cfg, self.cfg.head_dim
        P, ms = self.world, self.ms
        sv = {}
        sv["x"] = x
        sv["st1"] = self._norm_fwd(x, blk.g1, self.c_qkv.x_shard)
        sv["h1_full"] = torch.empty(P * ms, cfg.dim, device=x.device, dtype=torch.bfloat16)
        qkv = self.c_qkv.ag_gemm(blk.w_qkv.shadow, True, stage=sv["h1_full"])
        sv["h1_full"][self.rank * ms:(self.rank + 1) * ms].copy_(self.c_qkv.x_shard)
        q4 = qkv.view(self.B, self.S, blk.hq + 2 * blk.hkv, hd)
        q, k, v = q4[:, :, : blk.hq], q4[:, :, blk.hq: blk.hq + blk.hkv], q4[:, :, blk.hq + blk.hkv:]
        o, lse = flash_attention_forward(q, k, v, mask="block_causal", frame=cfg.frame_len)
        sv.update(qkv=qkv, o=o, lse=lse)
        x1 = self.c_out.gemm_rs(o.view(P * ms, blk.hq * hd), blk.w_out.shadow, True, residual=x)
        sv["x1"] = x1
        sv["st2"] = self._norm_fwd(x1, blk.g2, self.c_up.x_shard)
        sv["h2_full"] = torch.empty(P * ms, cfg.dim, device=x.device, dtype=torch.bfloat16)
        gu = self.c_up.ag_gemm(blk.w_up.shadow, True, stage=sv["h2_full"])
        sv["h2_full"][self.rank * ms:(self.rank + 1) * ms].copy_(self.c_up.x_shard)
        hmid = self._swiglu(gu, blk.ffl)
        sv.update(gu=gu, hmid=hmid)
        x2 = self.c_down.gemm_rs(hmid, blk.w_down.shadow, True, residual=x1)
        return x2, sv

    def _block_bwd(self, blk: TPBlock, sv, dx2):
        cfg, hd = self.cfg, self.cfg.head_dim
        P, ms = self.world, self.ms
        # ---- FFN down (row parallel): dhmid = gather(dx2) · W_downᵀ ; dW_down += hmidᵀ · gather(dx2)
        self.cb_down.x_shard.copy_(dx2)
        dhmid = self.cb_down.ag_gemm(blk.w_down.shadow, False)
        dy_full = self.cb_down.gathered_input()
        ops.gemm(sv["hmid"], dy_full, a_mn=True, b_mn=True, out=blk.w_down.grad_storage, accumulate=True)
        dgu = self._swiglu_bwd(sv["gu"], dhmid, blk.ffl)
        # ---- FFN up (column parallel): dh2 = reduce_scatter(dgu · W_upᵀ) ; dW_up += h2_fullᵀ · dgu
        ops.gemm(sv["h2_full"], dgu, a_mn=True, b_mn=True, out=blk.w_up.grad_storage, accumulate=True)
        dh2 = self.cb_up.gemm_rs(dgu, blk.w_up.shadow, False)
        dx1 = self._norm_bwd(sv["x1"], dh2, blk.g2, sv["st2"])
        dx1.add_(dx2)
        # ---- attention out (row parallel)
        self.cb_out.x_shard.copy_(dx1)
        do = self.cb_out.ag_gemm(blk.w_out.shadow, False)
        dy_full = self.cb_out.gathered_input()
        o2 = sv["o"].view(P * ms, blk.hq * hd)
        ops.gemm(o2, dy_full, a_mn=True, b_mn=True, out=blk.w_out.grad_storage, accumulate=True)
        # ---- attention core
        q4 = sv["qkv"].view(self.B, self.S, blk.hq + 2 * blk.hkv, hd)
        q, k, v = q4[:, :, : blk.hq], q4[:, :, blk.hq: blk.hq + blk.hkv], q4[:, :, blk.hq + blk.hkv:]
        dqkv = torch.empty_like(q4)
        flash_attention_backward(q, k, v, sv["o"], sv["lse"], do.view(self.B, self.S, blk.hq, hd), mask="block_causal",
                                 frame=cfg.frame_len, dq=dqkv[:, :, : blk.hq], dk=dqkv[:, :, blk.hq: blk.hq + blk.hkv],
                                 dv=dqkv[:, :, blk.hq + blk.hkv:])
        dqkv2 = dqkv.view(P * ms, -1)
        # ---- QKV (column parallel)
        ops.gemm(sv["h1_full"], dqkv2, a_mn=True, b_mn=True, out=blk.w_qkv.grad_storage, accumulate=True)
        dh1 = self.cb_qkv.gemm_rs(dqkv2, blk.w_qkv.shadow, False)
        dx = self._norm_bwd(sv["x"], dh1, blk.g1, sv["st1"])
        dx.add_(dx1)
        return dx

    # ------------------------------------------------------------------ full step
    def train_step(self, z1_shard, act_shard, noise_shard, t_rows):
        """One optimisation step on this rank's row shard.
        z1_shard / noise_shard: [Ms, latent_dim] fp32 (zero on non-latent rows), act_shard: [Ms, action_dim],
        t_rows: [Ms] flow time of the row's sequence.  Returns the device loss accumulator (summed loss)."""
        cfg = self.cfg
        ms = self.ms
        lat = self.is_lat[:, None]
        zt = ((1 - t_rows[:, None]) * noise_shard + t_rows[:, None] * z1_shard) * lat
        target = (z1_shard - noise_shard) * lat
        zt_b = torch.zeros(ms, 64, device=self.device, dtype=torch.bfloat16)
        zt_b[:, : cfg.latent_dim] = zt
        a_b = torch.zeros(ms, 64, device=self.device, dtype=torch.bfloat16)
        a_b[:, : cfg.action_dim] = act_shard * self.is_act[:, None]
        temb = nn.sincos_embed(t_rows, cfg.dim)
        x = self.in_lat.forward(zt_b) + self.in_act.forward(a_b) + self.t_lin.forward(temb) + self.pos
        saves = []
        for blk in self.blocks:
            x, sv = self._block_fwd(blk, x)
            saves.append(sv)
        hn = torch.empty_like(x)
        st = self._norm_fwd(x, self.out_g, hn)
        pred = self.out_lin.forward(hn)  # [Ms, 32]
        n_lat = float(self.B * cfg.frames * cfg.tokens_per_frame * cfg.latent_dim)
        dpred = torch.empty(ms, cfg.latent_dim, device=self.device, dtype=torch.bfloat16)
        check(self.lib.nb_mse_loss(ptr(pred), ctypes.c_int(pred.stride(0)), ptr(target.contiguous()), ctypes.c_int(cfg.latent_dim),
                                   ptr(self.is_lat), ptr(dpred), ctypes.c_int(cfg.latent_dim), ptr(self._ws), ptr(self.loss_acc),
                                   ctypes.c_int(ms), ctypes.c_int(cfg.latent_dim), ctypes.c_int(cfg.latent_dim),
                                   ctypes.c_float(1.0 / n_lat), ctypes.c_float(1.0 / n_lat), ctypes.c_int(0),
                                   ctypes.c_int(int(pred.dtype == torch.float32)), stream_ptr()), "mse")
        # ---- backward
        dhn = self.out_lin.vjp(dpred)
        dx = self._norm_bwd(x, dhn, self.out_g, st)
        for blk, sv in zip(reversed(self.blocks), reversed(saves)):
            dx = self._block_bwd(blk, sv, dx)
            sv.clear()
        self.in_lat.vjp(dx)
        self.in_act.vjp(dx)
        self.t_lin.vjp(dx)
        # ---- optimizer: KV replicas summed in their group, replicated params all-reduced + AdamW fused
        if self.kv_group is not None:
            q_cols = self.blocks[0].hq * cfg.head_dim
            kvw = self._kv_pack.shape[2]
            for i, blk in enumerate(self.blocks):
                self._kv_pack[i].copy_(blk.w_qkv.grad_storage[:, q_cols: q_cols + kvw])
            dist.all_reduce(self._kv_pack, group=self.kv_group)
            for i, blk in enumerate(self.blocks):
                blk.w_qkv.grad_storage[:, q_cols: q_cols + kvw].copy_(self._kv_pack[i])
        if self.grad_sync is not None:
            self.grad_sync.reduce_and_step(self.opt_rep)
        else:
            self.opt_rep.step(zero_grad=True)
        self.opt_shd.step(zero_grad=True)
        return self.loss_acc
