"""Export Qwen3.5 to the HuggingFace format, dense and MoE (reference:
omegalax/models/qwen3_5/params.py; the MoE branch writes the fused expert layout
``experts.gate_up_proj`` [E,2F,D] / ``experts.down_proj`` [E,D,F], the inverse of the loader)."""
from __future__ import annotations

from pathlib import Path

import torch

from ..hf_io import save_hf_config, torch_dtype_to_hf
from ..params_utils import save_safetensors, write_moe_experts_to_hf
from .config import Qwen3_5Config, Qwen3_5TextConfig


def qwen3_5_to_hf_config_dict(cfg) -> dict:
    if isinstance(cfg, Qwen3_5TextConfig):
        cfg = Qwen3_5Config(text_config=cfg)
    t, v = cfg.text_config, cfg.vision_config
    txt = {
        "model_type": "qwen3_5_moe_text" if t.is_moe else "qwen3_5_text",
        "vocab_size": t.vocab_size, "hidden_size": t.hidden_size, "num_hidden_layers": t.num_hidden_layers,
        "num_attention_heads": t.num_attention_heads, "num_key_value_heads": t.num_key_value_heads,
        "head_dim": t.head_dim, "rms_norm_eps": t.rms_norm_eps, "layer_types": list(t.layer_types),
        "attention_bias": t.attention_bias, "hidden_act": "silu", "dtype": torch_dtype_to_hf(t.dtype),
        "linear_conv_kernel_dim": t.linear_conv_kernel_dim, "linear_key_head_dim": t.linear_key_head_dim,
        "linear_num_key_heads": t.linear_num_key_heads, "linear_num_value_heads": t.linear_num_value_heads,
        "linear_value_head_dim": t.linear_value_head_dim, "full_attention_interval": 4,
        "rope_parameters": {"rope_type": "default", "rope_theta": t.rope_theta,
                            "partial_rotary_factor": t.partial_rotary_factor,
                            "mrope_section": list(t.mrope_section), "mrope_interleaved": t.mrope_interleaved},
    }
    if t.is_moe:
        txt.update(moe_intermediate_size=t.moe_intermediate_size,
                   shared_expert_intermediate_size=t.shared_expert_intermediate_size, num_experts=t.num_experts,
                   num_experts_per_tok=t.num_experts_per_tok, router_aux_loss_coef=t.router_aux_loss_coef)
    else:
        txt["intermediate_size"] = t.intermediate_size
    vis = {"model_type": "qwen3_5_moe_vision" if t.is_moe else "qwen3_5_vision" if False else "qwen3_5",
           "depth": v.depth, "hidden_size": v.hidden_size, "intermediate_size": v.intermediate_size,
           "num_heads": v.num_heads, "patch_size": v.patch_size, "temporal_patch_size": v.temporal_patch_size,
           "spatial_merge_size": v.spatial_merge_size, "in_channels": v.in_channels,
           "out_hidden_size": v.out_hidden_size, "num_position_embeddings": v.num_position_embeddings,
           "hidden_act": "gelu_pytorch_tanh", "dtype": torch_dtype_to_hf(v.dtype)}
    vis.pop("model_type")
    return {
        "architectures": ["Qwen3_5MoeForConditionalGeneration" if t.is_moe else "Qwen3_5ForConditionalGeneration"],
        "model_type": "qwen3_5_moe" if t.is_moe else "qwen3_5",
        "text_config": txt, "vision_config": vis, "tie_word_embeddings": t.tie_word_embeddings,
        "image_token_id": cfg.image_token_id, "video_token_id": cfg.video_token_id,
        "vision_start_token_id": cfg.vision_start_token_id, "vision_end_token_id": cfg.vision_end_token_id,
    }


def vision_to_hf_tensors(visual, vcfg, prefix: str = "model.visual") -> dict[str, torch.Tensor]:
    f32 = lambda t: t.detach().float().contiguous()  # noqa: E731
    out = {
        f"{prefix}.patch_embed.proj.weight": f32(visual.patch_embed.weight).reshape(
            vcfg.hidden_size, vcfg.in_channels, vcfg.temporal_patch_size, vcfg.patch_size, vcfg.patch_size),
        f"{prefix}.patch_embed.proj.bias": f32(visual.patch_embed.bias),
        f"{prefix}.pos_embed.weight": f32(visual.pos_embed),
    }
    for i, blk in enumerate(visual.blocks):
        for hf, mod in (("norm1", blk.norm1), ("norm2", blk.norm2), ("attn.qkv", blk.attn.qkv), ("attn.proj", blk.attn.proj),
                        ("mlp.linear_fc1", blk.mlp.linear_fc1), ("mlp.linear_fc2", blk.mlp.linear_fc2)):
            out[f"{prefix}.blocks.{i}.{hf}.weight"] = f32(mod.weight)
            out[f"{prefix}.blocks.{i}.{hf}.bias"] = f32(mod.bias)
    def merger(p, mg):
        for part in ("norm", "linear_fc1", "linear_fc2"):
            out[f"{p}.{part}.weight"] = f32(getattr(mg, part).weight)
            out[f"{p}.{part}.bias"] = f32(getattr(mg, part).bias)
    merger(f"{prefix}.merger", visual.merger)
    for i, mg in enumerate(visual.deepstack_mergers):
        merger(f"{prefix}.deepstack_merger_list.{i}", mg)
    return out


def text_to_hf_tensors(model, t: Qwen3_5TextConfig, prefix: str = "model.language_model") -> dict[str, torch.Tensor]:
    f32 = lambda x: x.detach().float().contiguous()  # noqa: E731
    H, G, K = t.num_attention_heads, t.num_key_value_heads, t.head_dim
    out = {f"{prefix}.embed_tokens.weight": f32(model.embedder.weight), f"{prefix}.norm.weight": f32(model.final_norm.weight)}
    for i, layer in enumerate(model.layers):
        p = f"{prefix}.layers.{i}"
        out[f"{p}.input_layernorm.weight"] = f32(layer.input_norm.weight)
        out[f"{p}.post_attention_layernorm.weight"] = f32(layer.post_norm.weight)
        if layer.layer_type == "full_attention":
            a = layer.attn
            w = a.qkv_proj.weight
            out[f"{p}.self_attn.q_proj.weight"] = f32(w[: 2 * H * K])
            out[f"{p}.self_attn.k_proj.weight"] = f32(w[2 * H * K:(2 * H + G) * K])
            out[f"{p}.self_attn.v_proj.weight"] = f32(w[(2 * H + G) * K:])
            out[f"{p}.self_attn.o_proj.weight"] = f32(a.o_proj.weight)
            if a.qkv_proj.bias is not None:
                b = a.qkv_proj.bias
                out[f"{p}.self_attn.q_proj.bias"] = f32(b[: 2 * H * K])
                out[f"{p}.self_attn.k_proj.bias"] = f32(b[2 * H * K:(2 * H + G) * K])
                out[f"{p}.self_attn.v_proj.bias"] = f32(b[(2 * H + G) * K:])
                out[f"{p}.self_attn.o_proj.bias"] = f32(a.o_proj.bias)
            out[f"{p}.self_attn.q_norm.weight"] = f32(a.q_norm.weight)
            out[f"{p}.self_attn.k_norm.weight"] = f32(a.k_norm.weight)
        else:
            d = layer.linear_attn
            for nm in ("in_proj_qkv", "in_proj_z", "in_proj_b", "in_proj_a", "out_proj"):
                out[f"{p}.linear_attn.{nm}.weight"] = f32(getattr(d, nm).weight)
            out[f"{p}.linear_attn.conv1d.weight"] = f32(d.conv_weight).unsqueeze(1)
            out[f"{p}.linear_attn.dt_bias"] = f32(d.dt_bias)
            out[f"{p}.linear_attn.A_log"] = f32(d.A_log)
            out[f"{p}.linear_attn.norm.weight"] = f32(d.norm.weight)
        if layer.is_moe:
            m = layer.mlp
            write_moe_experts_to_hf(out, p, m.router.weight, m.experts_gate_up, m.experts_down)
            Fs = t.shared_expert_intermediate_size
            gu = m.shared_expert.gate_up_proj.weight
            out[f"{p}.mlp.shared_expert.gate_proj.weight"] = f32(gu[:Fs])
            out[f"{p}.mlp.shared_expert.up_proj.weight"] = f32(gu[Fs:])
            out[f"{p}.mlp.shared_expert.down_proj.weight"] = f32(m.shared_expert.down_proj.weight)
            out[f"{p}.mlp.shared_expert_gate.weight"] = f32(m.shared_expert_gate.weight)
        else:
            F = t.intermediate_size
            gu = layer.mlp.gate_up_proj.weight
            out[f"{p}.mlp.gate_proj.weight"] = f32(gu[:F])
            out[f"{p}.mlp.up_proj.weight"] = f32(gu[F:])
            out[f"{p}.mlp.down_proj.weight"] = f32(layer.mlp.down_proj.weight)
    return out


def export_qwen3_5_to_safetensors(model, cfg, out_dir) -> Path:
    """Write ``model.safetensors`` + ``config.json``.  Accepts the conditional-generation
    model (with vision tower) or the text-only model."""
    full = isinstance(cfg, Qwen3_5Config)
    tcfg = cfg.text_config if full else cfg
    tensors = text_to_hf_tensors(model.model, tcfg)
    tensors["lm_head.weight"] = model.lm_head.weight.detach().float().contiguous()
    if full and hasattr(model, "visual"):
        tensors.update(vision_to_hf_tensors(model.visual, cfg.vision_config))
    save_safetensors(tensors, out_dir)
    save_hf_config(qwen3_5_to_hf_config_dict(cfg), out_dir)
    return Path(out_dir)
