"""Export Qwen3-VL to the HuggingFace format (reference: omegalax/models/qwen3_vl/params.py)."""
from __future__ import annotations

from pathlib import Path

from ..hf_io import save_hf_config, torch_dtype_to_hf
from ..params_utils import save_safetensors
from ..qwen3.params import decoder_to_hf_tensors
from ..qwen3_5.params import vision_to_hf_tensors
from .config import Qwen3VLConfig


def qwen3_vl_to_hf_config_dict(cfg: Qwen3VLConfig) -> dict:
    v = cfg.vision
    txt = {
        "model_type": "qwen3_vl_moe_text" if cfg.is_moe else "qwen3_vl_text",
        "num_hidden_layers": cfg.num_layers, "vocab_size": cfg.vocab_size, "hidden_size": cfg.emb_dim,
        "intermediate_size": cfg.mlp_dim, "num_attention_heads": cfg.num_heads, "head_dim": cfg.head_dim,
        "num_key_value_heads": cfg.num_kv_heads, "rms_norm_eps": cfg.norm_eps, "hidden_act": "silu",
        "attention_bias": False, "dtype": torch_dtype_to_hf(cfg.dtype), "rope_theta": cfg.rope_theta,
        "rope_scaling": {"rope_type": "default", "mrope_section": list(cfg.mrope_section), "mrope_interleaved": True},
        "rope_parameters": {"rope_type": "default", "rope_theta": cfg.rope_theta,
                            "mrope_section": list(cfg.mrope_section), "mrope_interleaved": True},
    }
    if cfg.is_moe:
        txt.update(moe_intermediate_size=cfg.moe_intermediate_size, num_experts=cfg.num_experts,
                   num_experts_per_tok=cfg.num_experts_per_tok, mlp_only_layers=list(cfg.mlp_only_layers),
                   decoder_sparse_step=cfg.decoder_sparse_step, norm_topk_prob=cfg.norm_topk_prob)
    vis = {"hidden_size": v.hidden_size, "intermediate_size": v.intermediate_size, "num_heads": v.num_heads,
           "patch_size": v.patch_size, "temporal_patch_size": v.temporal_patch_size, "in_channels": v.in_channels,
           "spatial_merge_size": v.spatial_merge_size, "out_hidden_size": v.out_hidden_size, "depth": v.depth,
           "hidden_act": v.hidden_act, "num_position_embeddings": v.num_position_embeddings,
           "deepstack_visual_indexes": list(v.deepstack_visual_indexes), "dtype": torch_dtype_to_hf(v.dtype)}
    out = {"architectures": ["Qwen3VLMoeForConditionalGeneration" if cfg.is_moe else "Qwen3VLForConditionalGeneration"],
           "model_type": "qwen3_vl_moe" if cfg.is_moe else "qwen3_vl", "text_config": txt, "vision_config": vis,
           "tie_word_embeddings": cfg.tie_word_embeddings, "image_token_id": cfg.image_token_id,
           "video_token_id": cfg.video_token_id, "vision_start_token_id": cfg.vision_start_token_id}
    if cfg.vision_end_token_id is not None:   # only what a loaded config said; never guessed
        out["vision_end_token_id"] = cfg.vision_end_token_id
    return out


def export_qwen3_vl_to_safetensors(model, cfg: Qwen3VLConfig, out_dir) -> Path:
    tensors = decoder_to_hf_tensors(model, cfg, "model.language_model")
    tensors["lm_head.weight"] = model.lm_head.weight.detach().float().contiguous()
    tensors.update(vision_to_hf_tensors(model.visual, cfg.vision))
    save_safetensors(tensors, out_dir)
    save_hf_config(qwen3_vl_to_hf_config_dict(cfg), out_dir)
    return Path(out_dir)
