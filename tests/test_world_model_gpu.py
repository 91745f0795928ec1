"""Tiny world model: the TP+SP code path at world = 1 against an fp32 PyTorch restatement of the same network."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_world_model_step_matches_torch_reference():
    from noeira_b200.models.world_model import WorldModel, WorldModelConfig
    from noeira_b200.ops import check_status
    cfg = WorldModelConfig(layers=2, dim=256, heads=2, kv_heads=1, head_dim=128, ff=512, frames=4, tokens_per_frame=31,
                           latent_dim=32, action_dim=6, lr=1e-3)
    B = 2
    m = WorldModel(cfg, batch=B)
    ms = m.ms
    g = torch.Generator(device="cuda").manual_seed(0)
    z1 = torch.randn(ms, 32, device="cuda", generator=g) * m.is_lat[:, None]
    nz = torch.randn(ms, 32, device="cuda", generator=g) * m.is_lat[:, None]
    act = torch.rand(ms, 6, device="cuda", generator=g) * 2 - 1
    t = torch.rand(B, device="cuda", generator=g).repeat_interleave(m.S)
    # ---- fp32 reference with autograd on copies of the parameters
    P = {n: p.data.clone().float().requires_grad_(True) for n, p in
         list(m.opt_rep.arena.entries and [(e[0], e[1]) for e in m.opt_rep.arena.entries])
         + [(e[0], e[1]) for e in m.opt_shd.arena.entries]}
    lat = m.is_lat[:, None]
    zt = ((1 - t[:, None]) * nz + t[:, None] * z1) * lat
    target = (z1 - nz) * lat
    from noeira_b200 import nn
    temb = nn.sincos_embed(t, cfg.dim).float()
    x = zt.bfloat16().float() @ P["in_latent.weight"] + (act * m.is_act[:, None]).bfloat16().float() @ P["in_action.weight"] \
        + torch.nn.functional.silu(temb @ P["time.weight"]) + m.pos.float()

    def rms(v, gam):
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-5) * gam

    S, hd = m.S, cfg.head_dim
    qi = torch.arange(S, device="cuda")
    ok = (qi[None, :] // cfg.frame_len) <= (qi[:, None] // cfg.frame_len)
    for i in range(cfg.layers):
        pre = f"blocks.{i}."
        h = rms(x, P[pre + "norm1.gamma"])
        qkv = (h @ P[pre + "attn.qkv.weight"]).view(B, S, 4, hd)
        q, k, v = qkv[:, :, :2], qkv[:, :, 2:3], qkv[:, :, 3:4]
        sc = torch.einsum("bqhd,bkhd->bhqk", q, k.expand(-1, -1, 2, -1)) / math.sqrt(hd)
        sc = sc.masked_fill(~ok, float("-inf"))
        o = torch.einsum("bhqk,bkhd->bqhd", sc.softmax(-1), v.expand(-1, -1, 2, -1)).reshape(B * S, 2 * hd)
        x = x + o @ P[pre + "attn.out.weight"]
        h = rms(x, P[pre + "norm2.gamma"])
        gu = h @ P[pre + "ffn.0.weight"]
        H = cfg.ff
        x = x + (torch.nn.functional.silu(gu[:, :H]) * gu[:, H:]) @ P[pre + "ffn.1.weight"]
    pred = rms(x, P["out_norm.gamma"]) @ P["out.weight"]
    n_lat = B * cfg.frames * cfg.tokens_per_frame * cfg.latent_dim
    loss = (((pred - target) * lat) ** 2).sum() / n_lat
    loss.backward()
    # ---- our step (gradients are consumed by the optimizer, so compare the parameter UPDATE direction instead)
    before = {e[0]: e[1].data.clone() for e in m.opt_rep.arena.entries + m.opt_shd.arena.entries}
    acc = m.train_step(z1, act, nz, t)
    torch.cuda.synchronize()
    check_status()
    assert abs(acc.item() - loss.item()) < 3e-2 * max(1.0, loss.item()), (acc.item(), loss.item())
    # first Adam step moves each weight by -lr * sign(g) (bias-corrected m/sqrt(v) = ±1): check the sign agreement
    agree, total = 0, 0
    for e in m.opt_rep.arena.entries + m.opt_shd.arena.entries:
        name, p = e[0], e[1]
        gref = P[name].grad
        big = gref.abs() > 0.2 * gref.abs().max()
        upd = (p.data - before[name])[big]
        agree += int((torch.sign(upd) == -torch.sign(gref[big])).sum())
        total += int(big.sum())
    assert agree / max(total, 1) > 0.97, (agree, total)
