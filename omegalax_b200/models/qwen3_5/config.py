"""Qwen3.5 configuration: hybrid GatedDeltaNet / gated-attention decoder (dense or MoE FFN)
plus a vision tower (reference: omegalax/models/qwen3_5/config.py)."""
from __future__ import annotations

import dataclasses
from pathlib import Path
from typing import Any

import torch

from ..hf_io import hf_dtype_to_torch, load_hf_config_from_source
from ..shard_config import ShardConfig

FULL_ATTENTION_INTERVAL = 4


@dataclasses.dataclass(frozen=True)
class Qwen3_5VisionConfig:
    depth: int = 27
    hidden_size: int = 1152
    intermediate_size: int = 4304
    num_heads: int = 16
    patch_size: int = 16
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    in_channels: int = 3
    out_hidden_size: int = 4096
    num_position_embeddings: int = 2304
    dtype: Any = torch.bfloat16


@dataclasses.dataclass(frozen=True)
class Qwen3_5TextConfig:
    vocab_size: int = 248_320
    hidden_size: int = 4096
    num_hidden_layers: int = 60
    num_attention_heads: int = 32
    num_key_value_heads: int = 2
    head_dim: int = 256
    rms_norm_eps: float = 1e-6
    layer_types: tuple[str, ...] = ()
    rope_theta: float = 10_000_000
    partial_rotary_factor: float = 0.25
    mrope_section: tuple[int, ...] = (11, 11, 10)
    mrope_interleaved: bool = True   # kept for config fidelity; the interleaved form is always used
    attention_bias: bool = False
    tie_word_embeddings: bool = False
    # GatedDeltaNet (linear attention)
    linear_conv_kernel_dim: int = 4
    linear_key_head_dim: int = 128
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 64
    linear_value_head_dim: int = 128
    # dense FFN (num_experts == 0)
    intermediate_size: int = 0
    # MoE FFN
    moe_intermediate_size: int = 0
    shared_expert_intermediate_size: int = 0
    num_experts: int = 0
    num_experts_per_tok: int = 0
    router_aux_loss_coef: float = 0.001
    shd_cfg: ShardConfig = dataclasses.field(default_factory=ShardConfig.default)
    dtype: Any = torch.bfloat16

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0


@dataclasses.dataclass(frozen=True)
class Qwen3_5Config:
    vision_config: Qwen3_5VisionConfig = dataclasses.field(default_factory=Qwen3_5VisionConfig)
    text_config: Qwen3_5TextConfig = dataclasses.field(default_factory=Qwen3_5TextConfig)
    image_token_id: int = 248_056
    video_token_id: int = 248_057
    vision_start_token_id: int = 248_053
    vision_end_token_id: int = 248_054


def generate_layer_types(num_layers: int) -> tuple[str, ...]:
    """Every fourth layer (1-indexed) is full attention, the rest are linear attention."""
    return tuple("full_attention" if (i + 1) % FULL_ATTENTION_INTERVAL == 0 else "linear_attention"
                 for i in range(num_layers))


_SMOKE_VISION = dict(depth=2, hidden_size=64, intermediate_size=128, num_heads=4, patch_size=16,
                     temporal_patch_size=2, spatial_merge_size=2, in_channels=3, out_hidden_size=128,
                     num_position_embeddings=100)
_SMOKE_TEXT = dict(vocab_size=1024, hidden_size=128, num_hidden_layers=4, num_attention_heads=4,
                   num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-6, layer_types=generate_layer_types(4),
                   rope_theta=10_000, partial_rotary_factor=0.25, mrope_section=(2, 1, 1),
                   linear_conv_kernel_dim=4, linear_key_head_dim=16, linear_num_key_heads=2,
                   linear_num_value_heads=4, linear_value_head_dim=32)
_SMOKE_SPECS: dict[str, dict[str, Any]] = {
    "qwen3.5-smoke": {"vision_config": _SMOKE_VISION,
                      "text_config": dict(_SMOKE_TEXT, moe_intermediate_size=64, shared_expert_intermediate_size=64,
                                          num_experts=4, num_experts_per_tok=2)},
    "qwen3.5-smoke-dense": {"vision_config": _SMOKE_VISION, "text_config": dict(_SMOKE_TEXT, intermediate_size=256)},
}

# The benchmark slice: the published 397B-A17B width truncated to 8 layers (3 GatedDeltaNet : 1
# gated attention, 512 experts top-10 + 1 shared expert of 1024, hidden 4096, vocabulary 248320).
_ARCH_SPECS: dict[str, dict[str, Any]] = {
    "qwen3.5-397b-a17b-8layer": {
        "vision_config": dict(),
        "text_config": dict(vocab_size=248_320, hidden_size=4096, num_hidden_layers=8, num_attention_heads=32,
                            num_key_value_heads=2, head_dim=256, layer_types=generate_layer_types(8),
                            rope_theta=10_000_000, partial_rotary_factor=0.25, mrope_section=(11, 11, 10),
                            linear_conv_kernel_dim=4, linear_key_head_dim=128, linear_num_key_heads=16,
                            linear_num_value_heads=64, linear_value_head_dim=128, moe_intermediate_size=1024,
                            shared_expert_intermediate_size=1024, num_experts=512, num_experts_per_tok=10),
    },
}

_REPOS = ("Qwen/Qwen3.5-0.8B", "Qwen/Qwen3.5-2B", "Qwen/Qwen3.5-4B", "Qwen/Qwen3.5-9B", "Qwen/Qwen3.5-27B",
          "Qwen/Qwen3.5-35B-A3B", "Qwen/Qwen3.5-122B-A10B", "Qwen/Qwen3.5-397B-A17B")
_SUPPORTED_MODEL_TYPES = {"qwen3_5", "qwen3_5_moe"}
_SUPPORTED_MODEL_IDS = sorted((*_SMOKE_SPECS, *_ARCH_SPECS, *_REPOS))


def list_qwen3_5_model_ids() -> list[str]:
    return list(_REPOS)


def list_supported_qwen3_5_model_ids() -> list[str]:
    return list(_SUPPORTED_MODEL_IDS)


def resolve_qwen3_5_repo_id(model_id: str) -> str:
    return model_id


def is_supported_qwen3_5_model_id(model_id: str) -> bool:
    return model_id in _SMOKE_SPECS or model_id in _ARCH_SPECS or model_id in _REPOS


def get_qwen3_5_spec(model_id: str) -> dict[str, Any]:
    if model_id in _SMOKE_SPECS:
        return dict(_SMOKE_SPECS[model_id])
    if model_id in _ARCH_SPECS:
        return dict(_ARCH_SPECS[model_id])
    if model_id in _REPOS:
        return {"hf_repo_id": model_id}
    raise ValueError(f"Unsupported Qwen3.5 model_id '{model_id}'. Supported ids: {_SUPPORTED_MODEL_IDS}")


def _req(m: dict, key: str, where: str):
    if key not in m:
        raise ValueError(f"Missing required key '{key}' in {where}.")
    return m[key]


def make_config(model_id: str) -> Qwen3_5Config:
    for table in (_SMOKE_SPECS, _ARCH_SPECS):
        if model_id in table:
            spec = table[model_id]
            return Qwen3_5Config(vision_config=Qwen3_5VisionConfig(**spec["vision_config"]),
                                 text_config=Qwen3_5TextConfig(**spec["text_config"]))
    if "/" not in model_id and not Path(model_id).expanduser().exists():
        raise ValueError(f"Unsupported Qwen3.5 model_id '{model_id}'. Supported ids: {_SUPPORTED_MODEL_IDS}")
    return make_config_from_hf(load_hf_config_from_source(resolve_qwen3_5_repo_id(model_id)))


def make_config_from_hf(hf_cfg: dict[str, Any]) -> Qwen3_5Config:
    """From a HuggingFace ``config.json``.  Requires ``text_config.rope_parameters`` and exactly
    one of the dense (``intermediate_size``) or MoE settings."""
    mt = _req(hf_cfg, "model_type", "hf_cfg")
    if mt not in _SUPPORTED_MODEL_TYPES:
        raise ValueError(f"Unsupported Qwen3.5 model_type '{mt}'. Expected one of {sorted(_SUPPORTED_MODEL_TYPES)}.")
    vis = _req(hf_cfg, "vision_config", "hf_cfg")
    txt = _req(hf_cfg, "text_config", "hf_cfg")
    if not isinstance(vis, dict) or not isinstance(txt, dict):
        raise ValueError("Expected vision_config and text_config to be dicts in hf_cfg.")
    W = "hf_cfg['text_config']"
    rp = _req(txt, "rope_parameters", W)
    if not isinstance(rp, dict):
        raise ValueError("Expected rope_parameters to be a dict in hf_cfg['text_config'].")
    if rp.get("rope_type", "default") != "default":
        raise ValueError(f"Unsupported rope_parameters.rope_type '{rp.get('rope_type')}' for Qwen3.5.")
    tdt = hf_dtype_to_torch(_req(txt, "dtype", W))
    vdt = hf_dtype_to_torch(vis["dtype"]) if vis.get("dtype") is not None else tdt
    moe = mt == "qwen3_5_moe"
    if moe == ("intermediate_size" in txt):
        raise ValueError("Qwen3.5 config must map cleanly to exactly one of dense or MoE text settings.")
    kw = {k: _req(txt, k, W) for k in (
        "vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
        "rms_norm_eps", "attention_bias", "linear_conv_kernel_dim", "linear_key_head_dim", "linear_num_key_heads",
        "linear_num_value_heads", "linear_value_head_dim")}
    kw.update(layer_types=tuple(_req(txt, "layer_types", W)), rope_theta=_req(rp, "rope_theta", "rope_parameters"),
              partial_rotary_factor=_req(rp, "partial_rotary_factor", "rope_parameters"),
              mrope_section=tuple(_req(rp, "mrope_section", "rope_parameters")),
              mrope_interleaved=_req(rp, "mrope_interleaved", "rope_parameters"),
              tie_word_embeddings=_req(hf_cfg, "tie_word_embeddings", "hf_cfg"), dtype=tdt)
    if moe:
        kw.update({k: _req(txt, k, W) for k in ("moe_intermediate_size", "shared_expert_intermediate_size",
                                                 "num_experts", "num_experts_per_tok", "router_aux_loss_coef")})
    else:
        kw["intermediate_size"] = _req(txt, "intermediate_size", W)
    V = "hf_cfg['vision_config']"
    vkw = {k: _req(vis, k, V) for k in ("depth", "hidden_size", "intermediate_size", "num_heads", "patch_size",
                                        "temporal_patch_size", "spatial_merge_size", "in_channels",
                                        "out_hidden_size", "num_position_embeddings")}
    return Qwen3_5Config(vision_config=Qwen3_5VisionConfig(dtype=vdt, **vkw), text_config=Qwen3_5TextConfig(**kw),
                         image_token_id=_req(hf_cfg, "image_token_id", "hf_cfg"),
                         video_token_id=_req(hf_cfg, "video_token_id", "hf_cfg"),
                         vision_start_token_id=_req(hf_cfg, "vision_start_token_id", "hf_cfg"),
                         vision_end_token_id=_req(hf_cfg, "vision_end_token_id", "hf_cfg"))
