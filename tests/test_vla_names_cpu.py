"""SmolVLA checkpoint names: save with the published names / layouts, load into a second model, coverage both ways."""
import numpy as np
import torch


def test_hf_smolvla_names_roundtrip(tmp_path):
    from noeira_b200.io.safetensors import SafeTensors
    from noeira_b200.models.vla import VLAConfig, VLAModel
    from noeira_b200.models.vla_names import load_hf_smolvla, save_hf_smolvla, smolvla_rules
    cfg = VLAConfig(image=64, vit_layers=1, lm_layers=2, vocab=128)
    a, b = VLAModel(cfg), VLAModel(cfg)
    g = torch.Generator().manual_seed(0)
    for _, p in a.named_params():
        p.set_(torch.randn(p.shape, generator=g))
    path = str(tmp_path / "model.safetensors")
    n = save_hf_smolvla(a, path)
    st = SafeTensors(path)
    names = set(st.names())
    assert n == len(names)
    hd = cfg.head_dim
    assert tuple(st.shape("model.vlm_with_expert.vlm.model.vision_model.encoder.layers.0.self_attn.k_proj.weight")) == (cfg.vit_dim, cfg.vit_dim)
    assert tuple(st.shape("model.vlm_with_expert.vlm.model.text_model.layers.1.self_attn.v_proj.weight")) == (cfg.kv_heads * hd, cfg.hidden)
    assert tuple(st.shape("model.vlm_with_expert.vlm.model.vision_model.embeddings.patch_embedding.weight")) == (cfg.vit_dim, 3, cfg.patch, cfg.patch)
    assert tuple(st.shape("model.vlm_with_expert.lm_expert.layers.1.self_attn.k_proj.weight")) == (cfg.kv_heads * hd, cfg.kv_heads * hd)
    assert tuple(st.shape("model.action_time_mlp_in.weight")) == (cfg.expert_width, 2 * cfg.expert_width)
    # their q_proj is the transposed first block of our fused qkv
    ours = dict(a.named_params())["text_model.layers.0.attn.qkv.weight"].data
    q = st.get("model.vlm_with_expert.vlm.model.text_model.layers.0.self_attn.q_proj.weight")
    assert np.allclose(q, ours[:, : cfg.heads * hd].t().numpy())
    rep = load_hf_smolvla(b, path)
    assert not rep.unmapped and not rep.missing and not rep.unclaimed and len(rep.loaded) == len(list(b.named_params()))
    for (na, pa), (_, pb) in zip(a.named_params(), b.named_params()):
        assert torch.equal(pa.data, pb.data), na
    assert set(smolvla_rules(cfg)) == {n_ for n_, _ in a.named_params()}
