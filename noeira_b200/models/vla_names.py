"""Hugging Face SmolVLA checkpoint names ↔ the parameters of ``models.vla.VLAModel``.

The published checkpoint (``model.vlm_with_expert.{vlm.model.vision_model, vlm.model.text_model, lm_expert}.…`` plus the
top-level action heads ``model.state_proj`` …) stores every projection as its own ``torch.nn.Linear`` (``[out, in]``);
this framework fuses q / k / v into one ``qkv`` weight and gate / up into ``ffn.0`` (``[in, out]`` with the parts side by
side as columns), and runs the SigLIP patch convolution as a Linear over flattened ``(c, ph, pw)`` patches.  A rule maps
ONE of our parameters to one or several of their tensors (transposed and concatenated along our column axis).
Coverage is checked on both sides, as ``nn.torch_names`` does: a parameter without a rule, a rule whose tensor is
missing, and file tensors that no rule names are all reported.
Reference: noeira/deep_agents/smolvla/names.mojo:51-330 (vision / text / expert / heads name maps).
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import numpy as np
import torch

from ..io.safetensors import SafeTensors, SafeTensorsWriter
from ..nn.torch_names import TorchLoadReport, TorchNameError

VLM = "model.vlm_with_expert.vlm."
VISION = VLM + "model.vision_model."
TEXT = VLM + "model.text_model."
EXPERT = "model.vlm_with_expert.lm_expert."
HEADS = "model."

# a rule: our name → list of (their name, their shape, kind); kinds: "linear" = their [out, in] transposed into our
# columns, "plain" = same layout, "conv" = their [D, 3, P, P] flattened to our [3·P·P, D]
Rule = List[Tuple[str, Tuple[int, ...], str]]


def smolvla_rules(cfg) -> Dict[str, Rule]:
    c = cfg
    hd = c.head_dim
    kvw = c.kv_heads * hd
    qw = c.heads * hd
    R: Dict[str, Rule] = {}
    lin = lambda name, o, i: (name, (o, i), "linear")
    # ---- SigLIP tower
    g = (c.image // c.patch) ** 2
    R["vision_model.patch_embed.weight"] = [(VISION + "embeddings.patch_embedding.weight", (c.vit_dim, 3, c.patch, c.patch), "conv")]
    R["vision_model.patch_embed.bias"] = [(VISION + "embeddings.patch_embedding.bias", (c.vit_dim,), "plain")]
    R["vision_model.pos_embed"] = [(VISION + "embeddings.position_embedding.weight", (g, c.vit_dim), "plain")]
    for i in range(c.vit_layers):
        o, t = f"vision_model.layers.{i}.", VISION + f"encoder.layers.{i}."
        R[o + "norm1.gamma"] = [(t + "layer_norm1.weight", (c.vit_dim,), "plain")]
        R[o + "norm1.beta"] = [(t + "layer_norm1.bias", (c.vit_dim,), "plain")]
        R[o + "attn.qkv.weight"] = [lin(t + f"self_attn.{p}_proj.weight", c.vit_dim, c.vit_dim) for p in "qkv"]
        R[o + "attn.qkv.bias"] = [(t + f"self_attn.{p}_proj.bias", (c.vit_dim,), "plain") for p in "qkv"]
        R[o + "attn.out.weight"] = [lin(t + "self_attn.out_proj.weight", c.vit_dim, c.vit_dim)]
        R[o + "attn.out.bias"] = [(t + "self_attn.out_proj.bias", (c.vit_dim,), "plain")]
        R[o + "norm2.gamma"] = [(t + "layer_norm2.weight", (c.vit_dim,), "plain")]
        R[o + "norm2.beta"] = [(t + "layer_norm2.bias", (c.vit_dim,), "plain")]
        R[o + "ffn.0.weight"] = [lin(t + "mlp.fc1.weight", c.vit_ff, c.vit_dim)]
        R[o + "ffn.0.bias"] = [(t + "mlp.fc1.bias", (c.vit_ff,), "plain")]
        R[o + "ffn.1.weight"] = [lin(t + "mlp.fc2.weight", c.vit_dim, c.vit_ff)]
        R[o + "ffn.1.bias"] = [(t + "mlp.fc2.bias", (c.vit_dim,), "plain")]
    R["vision_model.post_norm.gamma"] = [(VISION + "post_layernorm.weight", (c.vit_dim,), "plain")]
    R["vision_model.post_norm.beta"] = [(VISION + "post_layernorm.bias", (c.vit_dim,), "plain")]
    R["vision_model.connector.weight"] = [lin(VLM + "model.connector.modality_projection.proj.weight", c.hidden,
                                               c.vit_dim * c.shuffle ** 2)]
    # ---- SmolLM2 tower
    R["text_model.embed_tokens.weight"] = [(TEXT + "embed_tokens.weight", (c.vocab, c.hidden), "plain")]
    for i in range(c.lm_layers):
        o, t = f"text_model.layers.{i}.", TEXT + f"layers.{i}."
        R[o + "norm1.gamma"] = [(t + "input_layernorm.weight", (c.hidden,), "plain")]
        R[o + "attn.qkv.weight"] = [lin(t + "self_attn.q_proj.weight", qw, c.hidden), lin(t + "self_attn.k_proj.weight", kvw, c.hidden),
                                    lin(t + "self_attn.v_proj.weight", kvw, c.hidden)]
        R[o + "attn.out.weight"] = [lin(t + "self_attn.o_proj.weight", c.hidden, qw)]
        R[o + "norm2.gamma"] = [(t + "post_attention_layernorm.weight", (c.hidden,), "plain")]
        R[o + "ffn.0.weight"] = [lin(t + "mlp.gate_proj.weight", c.ff, c.hidden), lin(t + "mlp.up_proj.weight", c.ff, c.hidden)]
        R[o + "ffn.1.weight"] = [lin(t + "mlp.down_proj.weight", c.hidden, c.ff)]
    # ---- action expert: even layers attend [prefix; suffix] (k / v from its own width), odd layers cross-attend the
    # prefix keys / values (k / v from the VLM's KV width)
    W = c.expert_width
    for i in range(c.lm_layers):
        o, t = f"lm_expert.layers.{i}.", EXPERT + f"layers.{i}."
        kv_in = W if i % 2 == 0 else kvw
        R[o + "input_layernorm.gamma"] = [(t + "input_layernorm.weight", (W,), "plain")]
        R[o + "self_attn.q_proj.weight"] = [lin(t + "self_attn.q_proj.weight", qw, W)]
        R[o + "self_attn.k_proj.weight"] = [lin(t + "self_attn.k_proj.weight", kvw, kv_in)]
        R[o + "self_attn.v_proj.weight"] = [lin(t + "self_attn.v_proj.weight", kvw, kv_in)]
        R[o + "self_attn.o_proj.weight"] = [lin(t + "self_attn.o_proj.weight", W, qw)]
        R[o + "post_attention_layernorm.gamma"] = [(t + "post_attention_layernorm.weight", (W,), "plain")]
        R[o + "mlp.0.weight"] = [lin(t + "mlp.gate_proj.weight", c.expert_ff, W), lin(t + "mlp.up_proj.weight", c.expert_ff, W)]
        R[o + "mlp.1.weight"] = [lin(t + "mlp.down_proj.weight", W, c.expert_ff)]
    R["lm_expert.norm.gamma"] = [(EXPERT + "norm.weight", (W,), "plain")]
    # ---- heads
    for ours, theirs, o_, i_ in (("state_proj", "state_proj", c.hidden, c.action_pad), ("action_in_proj", "action_in_proj", W, c.action_pad),
                                 ("action_out_proj", "action_out_proj", c.action_pad, W),
                                 ("action_time_mlp_in", "action_time_mlp_in", W, 2 * W), ("action_time_mlp_out", "action_time_mlp_out", W, W)):
        R[ours + ".weight"] = [lin(HEADS + theirs + ".weight", o_, i_)]
        R[ours + ".bias"] = [(HEADS + theirs + ".bias", (o_,), "plain")]
    return R


def _to_ours(arr: np.ndarray, kind: str) -> torch.Tensor:
    t = torch.from_numpy(np.asarray(arr, dtype=np.float32).copy())
    if kind == "linear":
        return t.t().contiguous()
    if kind == "conv":
        return t.reshape(t.shape[0], -1).t().contiguous()
    return t


def load_hf_smolvla(model, file) -> TorchLoadReport:
    st = file if isinstance(file, SafeTensors) else SafeTensors(file)
    rules = smolvla_rules(model.c)
    rep = TorchLoadReport("")
    have, claimed = set(st.names()), set()
    for name, p in model.named_params():
        rule = rules.get(name)
        if rule is None:
            rep.unmapped.append(name)
            continue
        parts = []
        for their, shape, kind in rule:
            if their not in have:
                rep.missing.append(their)
                break
            if tuple(st.shape(their)) != tuple(shape):
                raise TorchNameError(f"load_hf_smolvla: '{their}' has shape {list(st.shape(their))} but the rule declares {list(shape)}")
            claimed.add(their)
            parts.append(_to_ours(st.get(their), kind))
        else:
            v = parts[0] if len(parts) == 1 else torch.cat(parts, dim=-1)
            if tuple(v.shape) != tuple(p.shape):
                raise TorchNameError(f"load_hf_smolvla: '{name}' is {list(p.shape)}, its rule assembles {list(v.shape)}")
            p.set_(v)
            rep.loaded.append(name)
    rep.unclaimed = sorted(have - claimed)
    return rep


def save_hf_smolvla(model, path: str, dtype: str = "f32") -> int:
    rules = smolvla_rules(model.c)
    w = SafeTensorsWriter()
    w.add_metadata("producer", "noeira_b200")
    n = 0
    for name, p in model.named_params():
        rule = rules.get(name)
        if rule is None:
            raise TorchNameError(f"save_hf_smolvla: no rule for '{name}'")
        t = p.data.detach().float().cpu()
        col = 0
        for their, shape, kind in rule:
            if kind == "linear":
                part = t[:, col: col + shape[0]].t()
                col += shape[0]
            elif kind == "conv":
                part = t.t().reshape(shape)
            else:
                width = shape[-1] if t.dim() == 1 else None
                part = t[col: col + shape[0]] if (t.dim() == 1 and len(rule) > 1) else t
                col += shape[0] if t.dim() == 1 else 0
            arr = np.ascontiguousarray(part.numpy()).reshape(shape)
            (w.add_bf16 if dtype == "bf16" else w.add_f32)(their, arr, list(shape))
            n += 1
    w.write(path)
    return n
