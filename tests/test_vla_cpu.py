"""VLA on CPU (tiny config): expert VJP vs finite differences; prefix mask; Euler sampler shape."""
import torch


def _tiny():
    from noeira_b200.models.vla import VLAConfig
    return VLAConfig(image=32, patch=8, n_cam=2, vit_dim=32, vit_heads=2, vit_ff=64, vit_layers=1, shuffle=2, hidden=64,
                     heads=4, kv_heads=2, head_dim=16, ff=96, lm_layers=2, vocab=50, n_lang=5, expert_width=48, expert_ff=64,
                     chunk=6, action_dim=3, action_pad=8, lr=1e-3)


def test_vla_expert_vjp_and_sampler():
    from noeira_b200.models.vla import VLAModel
    c = _tiny()
    torch.manual_seed(0)
    m = VLAModel(c)
    B = 2
    img = torch.rand(B, c.n_cam, 3, 32, 32)
    ids = torch.randint(0, 50, (B, 5))
    state = torch.randn(B, 8)
    assert c.prefix_len == 2 * 4 + 5 + 1
    mask = m.prefix_mask(torch.device("cpu"))
    assert torch.isinf(mask[0, -1]) and mask[-1, 0] == 0 and mask[-1, -1] == 0
    kv = m.prefix(img, ids, state)
    assert len(kv) == 2 and kv[0][0].shape == (B, c.prefix_len, 2, 16)
    x_t, t = torch.randn(B, 6, 8), torch.rand(B)
    tgt = torch.randn(B, 6, 8)

    def loss():
        v = m.denoise(kv, x_t, t)
        return ((v - tgt)[..., :3] ** 2).mean().item(), v

    l0, v = loss()
    dv = torch.zeros_like(v)
    dv[..., :3] = 2 * (v - tgt)[..., :3] / (B * 6 * 3)
    m.denoise_vjp(dv)
    P = dict(m.named_params())
    for name, idx in [("lm_expert.layers.0.self_attn.q_proj.weight", (3, 5)), ("lm_expert.layers.1.self_attn.k_proj.weight", (2, 7)),
                      ("lm_expert.layers.1.mlp.0.weight", (4, 9)), ("action_in_proj.weight", (1, 2)),
                      ("action_time_mlp_in.weight", (50, 3)), ("action_out_proj.weight", (5, 1)),
                      ("lm_expert.layers.0.self_attn.v_proj.weight", (6, 6))]:
        p = P[name]
        e = 1e-3
        p.data[idx] += e
        lp = loss()[0]
        p.data[idx] -= 2 * e
        lm = loss()[0]
        p.data[idx] += e
        fd, g = (lp - lm) / (2 * e), p.grad[idx].item()
        assert abs(fd - g) < 5e-2 * max(abs(fd), abs(g)) + 2e-4, (name, g, fd)
    a = m.sample_actions(img, ids, state, steps=10, generator=torch.Generator().manual_seed(0))
    assert a.shape == (B, 6, 3) and torch.isfinite(a).all()
    names = [n for n, _ in m.trainable()]
    assert not any(n.startswith(("vision_model", "text_model")) for n in names) and "state_proj.weight" in names
