"""Export Qwen3 to the HuggingFace format (reference: omegalax/models/qwen3/params.py)."""
from __future__ import annotations

from pathlib import Path

import torch

from ..hf_io import save_hf_config, torch_dtype_to_hf
from ..params_utils import save_safetensors, write_moe_experts_to_hf
from .config import Qwen3Config
from .model import Qwen3


def qwen3_to_hf_config_dict(cfg: Qwen3Config) -> dict:
    d = {
        "architectures": ["Qwen3MoeForCausalLM" if cfg.is_moe else "Qwen3ForCausalLM"],
        "model_type": "qwen3_moe" if cfg.is_moe else "qwen3",
        "num_hidden_layers": cfg.num_layers,
        "vocab_size": cfg.vocab_size,
        "hidden_size": cfg.emb_dim,
        "intermediate_size": cfg.mlp_dim,
        "num_attention_heads": cfg.num_heads,
        "num_key_value_heads": cfg.num_kv_heads,
        "head_dim": cfg.head_dim,
        "rms_norm_eps": cfg.norm_eps,
        "tie_word_embeddings": cfg.tie_word_embeddings,
        "hidden_act": "silu",
        "attention_bias": False,
        "rope_theta": cfg.rope_theta,
        "rope_parameters": {"rope_type": "default", "rope_theta": cfg.rope_theta},
        "dtype": torch_dtype_to_hf(cfg.dtype),
        "max_position_embeddings": 40960,
    }
    if cfg.rope_scaling_factor is not None:
        d["rope_parameters"]["factor"] = cfg.rope_scaling_factor
    if cfg.local_rope_theta is not None:
        d["rope_parameters"]["local_rope_theta"] = cfg.local_rope_theta
    if cfg.is_moe:
        d.update(moe_intermediate_size=cfg.moe_intermediate_size, num_experts=cfg.num_experts,
                 num_experts_per_tok=cfg.num_experts_per_tok, mlp_only_layers=list(cfg.mlp_only_layers),
                 decoder_sparse_step=cfg.decoder_sparse_step, norm_topk_prob=cfg.norm_topk_prob,
                 router_aux_loss_coef=cfg.aux_loss_coef)
    return d


def decoder_to_hf_tensors(model, cfg, prefix: str = "model") -> dict[str, torch.Tensor]:
    """Native decoder parameters -> HF tensors (fp32)."""
    H, G, K, F = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.mlp_dim
    f32 = lambda t: t.detach().float().contiguous()  # noqa: E731
    out = {f"{prefix}.embed_tokens.weight": f32(model.embedder.weight)}
    for i, layer in enumerate(model.layers):
        p = f"{prefix}.layers.{i}"
        qkv = layer.attn.qkv_proj.weight
        out[f"{p}.self_attn.q_proj.weight"] = f32(qkv[: H * K])
        out[f"{p}.self_attn.k_proj.weight"] = f32(qkv[H * K:(H + G) * K])
        out[f"{p}.self_attn.v_proj.weight"] = f32(qkv[(H + G) * K:])
        out[f"{p}.self_attn.o_proj.weight"] = f32(layer.attn.o_proj.weight)
        out[f"{p}.self_attn.q_norm.weight"] = f32(layer.attn.q_norm.weight)
        out[f"{p}.self_attn.k_norm.weight"] = f32(layer.attn.k_norm.weight)
        out[f"{p}.input_layernorm.weight"] = f32(layer.input_norm.weight)
        out[f"{p}.post_attention_layernorm.weight"] = f32(layer.post_norm.weight)
        if layer.is_moe:
            write_moe_experts_to_hf(out, p, layer.mlp.router.weight, layer.mlp.experts_gate_up, layer.mlp.experts_down)
        else:
            gu = layer.mlp.gate_up_proj.weight
            out[f"{p}.mlp.gate_proj.weight"] = f32(gu[:F])
            out[f"{p}.mlp.up_proj.weight"] = f32(gu[F:])
            out[f"{p}.mlp.down_proj.weight"] = f32(layer.mlp.down_proj.weight)
    out[f"{prefix}.norm.weight"] = f32(model.final_norm.weight)
    return out


def export_qwen3_to_safetensors(model: Qwen3, cfg: Qwen3Config, out_dir) -> Path:
    """Write ``model.safetensors`` (fp32) and ``config.json`` in the HF layout."""
    tensors = decoder_to_hf_tensors(model, cfg, "model")
    tensors["lm_head.weight"] = model.lm_head.weight.detach().float().contiguous()
    save_safetensors(tensors, out_dir)
    save_hf_config(qwen3_to_hf_config_dict(cfg), out_dir)
    return Path(out_dir)
