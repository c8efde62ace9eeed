"""Qwen3-VL configuration (reference: omegalax/models/qwen3_vl/config.py)."""
from __future__ import annotations

import dataclasses
from pathlib import Path
from typing import Any

import torch

from ..hf_io import hf_dtype_to_torch, load_hf_config_from_source
from ..shard_config import ShardConfig


@dataclasses.dataclass(frozen=True)
class Qwen3VLVisionConfig:
    hidden_size: int
    intermediate_size: int
    num_heads: int
    patch_size: int
    temporal_patch_size: int
    in_channels: int
    spatial_merge_size: int
    out_hidden_size: int
    depth: int
    hidden_act: str
    num_position_embeddings: int
    deepstack_visual_indexes: tuple[int, ...]
    dtype: Any = torch.bfloat16


@dataclasses.dataclass(frozen=True)
class Qwen3VLConfig:
    num_layers: int
    vocab_size: int
    emb_dim: int
    mlp_dim: int
    num_heads: int
    head_dim: int
    num_kv_heads: int
    rope_theta: float
    norm_eps: float
    tie_word_embeddings: bool
    mrope_section: tuple[int, ...]
    vision: Qwen3VLVisionConfig
    image_token_id: int
    video_token_id: int
    vision_start_token_id: int
    vision_end_token_id: int | None = None   # carried through from a loaded HF config; not used by the model
    moe_intermediate_size: int = 0
    num_experts: int = 0
    num_experts_per_tok: int = 0
    mlp_only_layers: tuple[int, ...] = ()
    decoder_sparse_step: int = 1
    norm_topk_prob: bool = True
    shd_cfg: ShardConfig = dataclasses.field(default_factory=ShardConfig.default)
    dtype: Any = torch.bfloat16

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    def is_moe_layer(self, layer_idx: int) -> bool:
        return (self.num_experts > 0 and layer_idx not in self.mlp_only_layers
                and (layer_idx + 1) % self.decoder_sparse_step == 0)


def _smoke_vision(inter: int) -> dict:
    return dict(hidden_size=64, intermediate_size=inter, num_heads=4, patch_size=14, temporal_patch_size=2,
                in_channels=3, spatial_merge_size=2, out_hidden_size=128, depth=2, hidden_act="gelu_pytorch_tanh",
                num_position_embeddings=256, deepstack_visual_indexes=(0,))


_TEXT_SMOKE = dict(vocab_size=1024, emb_dim=128, mlp_dim=512, num_layers=2, num_heads=4, head_dim=32,
                   rope_theta=1_000_000, norm_eps=1e-6, tie_word_embeddings=False, mrope_section=(8, 4, 4),
                   image_token_id=2, video_token_id=3, vision_start_token_id=4)
_SMOKE_SPECS: dict[str, dict[str, Any]] = {
    "qwen3-vl-smoke": dict(_TEXT_SMOKE, num_kv_heads=4, vision=_smoke_vision(256)),
    "qwen3-vl-smoke-moe": dict(_TEXT_SMOKE, num_kv_heads=2, vision=_smoke_vision(128), moe_intermediate_size=128,
                               num_experts=4, num_experts_per_tok=2),
}
# Architecture of the published 2B checkpoint (public HF config values), so the benchmark can
# build it with random weights when no config.json is on disk.
_ARCH_SPECS: dict[str, dict[str, Any]] = {
    "Qwen/Qwen3-VL-2B-Instruct": dict(
        vocab_size=151936, emb_dim=2048, mlp_dim=6144, num_layers=28, num_heads=16, head_dim=128, num_kv_heads=8,
        rope_theta=5_000_000, norm_eps=1e-6, tie_word_embeddings=True, mrope_section=(24, 20, 20),
        image_token_id=151655, video_token_id=151656, vision_start_token_id=151652,
        vision=dict(hidden_size=1024, intermediate_size=4096, num_heads=16, patch_size=16, temporal_patch_size=2,
                    in_channels=3, spatial_merge_size=2, out_hidden_size=2048, depth=24,
                    hidden_act="gelu_pytorch_tanh", num_position_embeddings=2304,
                    deepstack_visual_indexes=(5, 11, 17))),
}
_REPOS = ("Qwen/Qwen3-VL-2B-Instruct", "Qwen/Qwen3-VL-30B-A3B-Instruct")
_SUPPORTED_MODEL_TYPES = {"qwen3_vl", "qwen3_vl_moe"}
_SUPPORTED_MODEL_IDS = sorted((*_SMOKE_SPECS, *_REPOS))


def list_qwen3_vl_model_ids() -> list[str]:
    return list(_REPOS)


def list_supported_qwen3_vl_model_ids() -> list[str]:
    return list(_SUPPORTED_MODEL_IDS)


def resolve_qwen3_vl_repo_id(model_id: str) -> str:
    return model_id


def is_supported_qwen3_vl_model_id(model_id: str) -> bool:
    return model_id in _SMOKE_SPECS or model_id in _REPOS


def get_vl_spec(model_id: str) -> dict[str, Any]:
    if model_id in _SMOKE_SPECS:
        return dict(_SMOKE_SPECS[model_id])
    if model_id in _REPOS:
        return {"hf_repo_id": model_id}
    raise ValueError(f"Unsupported Qwen3-VL model_id '{model_id}'. Supported ids: {_SUPPORTED_MODEL_IDS}")


def _from_spec(spec: dict) -> Qwen3VLConfig:
    spec = dict(spec)
    vis = dict(spec.pop("vision"))
    vis["deepstack_visual_indexes"] = tuple(vis["deepstack_visual_indexes"])
    spec["mrope_section"] = tuple(spec["mrope_section"])
    return Qwen3VLConfig(vision=Qwen3VLVisionConfig(**vis), **spec)


def make_vl_config(model_id: str) -> Qwen3VLConfig:
    if model_id in _SMOKE_SPECS:
        return _from_spec(_SMOKE_SPECS[model_id])
    if "/" not in model_id and not Path(model_id).expanduser().exists():
        raise ValueError(f"Unsupported Qwen3-VL model_id '{model_id}'. Supported ids: {_SUPPORTED_MODEL_IDS}")
    try:
        return make_vl_config_from_hf(load_hf_config_from_source(resolve_qwen3_vl_repo_id(model_id)))
    except (ValueError, FileNotFoundError):
        if model_id in _ARCH_SPECS:
            return _from_spec(_ARCH_SPECS[model_id])
        raise


def _req(m: dict, k: str, where: str):
    if k not in m:
        raise ValueError(f"Missing required key '{k}' in {where}.")
    return m[k]


def make_vl_config_from_hf(hf_cfg: dict[str, Any]) -> Qwen3VLConfig:
    """From a HuggingFace config.json.  The rope settings are accepted in both spellings: the
    legacy ``text_config.rope_theta`` + ``rope_scaling{mrope_section}`` and the transformers-5
    ``text_config.rope_parameters{rope_theta, mrope_section}``."""
    mt = _req(hf_cfg, "model_type", "hf_cfg")
    if mt not in _SUPPORTED_MODEL_TYPES:
        raise ValueError(f"Unsupported Qwen3-VL model_type '{mt}'. Expected one of {sorted(_SUPPORTED_MODEL_TYPES)}.")
    vis = _req(hf_cfg, "vision_config", "hf_cfg")
    txt = _req(hf_cfg, "text_config", "hf_cfg")
    if not isinstance(vis, dict) or not isinstance(txt, dict):
        raise ValueError("Expected vision_config and text_config to be dicts in hf_cfg.")
    T = "hf_cfg['text_config']"
    rp = txt.get("rope_parameters")
    if isinstance(rp, dict):
        rope_theta = _req(rp, "rope_theta", T + ".rope_parameters")
        scaling = rp
    else:
        rope_theta = _req(txt, "rope_theta", T)
        scaling = _req(txt, "rope_scaling", T)
        if not isinstance(scaling, dict):
            raise ValueError("Expected rope_scaling to be a dict in hf_cfg['text_config'].")
    if scaling.get("rope_type", "default") != "default":
        raise ValueError(f"Unsupported rope_type '{scaling.get('rope_type')}' for Qwen3-VL.")
    sec = _req(scaling, "mrope_section", T + ".rope_scaling")
    tdt = hf_dtype_to_torch(_req(txt, "dtype", T))
    vdt = hf_dtype_to_torch(vis["dtype"]) if vis.get("dtype") is not None else tdt
    moe = mt == "qwen3_vl_moe"
    V = "hf_cfg['vision_config']"
    vkw = {k: _req(vis, k, V) for k in ("hidden_size", "intermediate_size", "num_heads", "patch_size",
                                        "temporal_patch_size", "in_channels", "spatial_merge_size", "out_hidden_size",
                                        "depth", "hidden_act", "num_position_embeddings")}
    return Qwen3VLConfig(
        num_layers=_req(txt, "num_hidden_layers", T), vocab_size=_req(txt, "vocab_size", T),
        emb_dim=_req(txt, "hidden_size", T), mlp_dim=_req(txt, "intermediate_size", T),
        num_heads=_req(txt, "num_attention_heads", T), head_dim=_req(txt, "head_dim", T),
        num_kv_heads=_req(txt, "num_key_value_heads", T), rope_theta=rope_theta, norm_eps=_req(txt, "rms_norm_eps", T),
        tie_word_embeddings=_req(hf_cfg, "tie_word_embeddings", "hf_cfg"), mrope_section=tuple(sec),
        moe_intermediate_size=_req(txt, "moe_intermediate_size", T) if moe else 0,
        num_experts=(txt["num_experts"] if "num_experts" in txt else _req(txt, "num_local_experts", T)) if moe else 0,
        num_experts_per_tok=_req(txt, "num_experts_per_tok", T) if moe else 0,
        mlp_only_layers=tuple(txt.get("mlp_only_layers", ())) if moe else (),
        decoder_sparse_step=txt.get("decoder_sparse_step", 1) if moe else 1,
        norm_topk_prob=txt.get("norm_topk_prob", True) if moe else True,
        image_token_id=_req(hf_cfg, "image_token_id", "hf_cfg"), video_token_id=_req(hf_cfg, "video_token_id", "hf_cfg"),
        vision_start_token_id=_req(hf_cfg, "vision_start_token_id", "hf_cfg"),
        vision_end_token_id=hf_cfg.get("vision_end_token_id"), dtype=tdt,
        vision=Qwen3VLVisionConfig(deepstack_visual_indexes=tuple(_req(vis, "deepstack_visual_indexes", V)), dtype=vdt, **vkw))
