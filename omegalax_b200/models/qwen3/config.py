"""Qwen3 configuration, dense and mixture-of-experts (reference: omegalax/models/qwen3/config.py)."""
from __future__ import annotations

import dataclasses
from pathlib import Path
from typing import Any

import torch

from ..hf_io import hf_dtype_to_torch, load_hf_config_from_source
from ..shard_config import ShardConfig


@dataclasses.dataclass(frozen=True)
class Qwen3Config:
    num_layers: int
    vocab_size: int
    emb_dim: int
    mlp_dim: int
    num_heads: int
    head_dim: int
    num_kv_heads: int
    rope_theta: float
    rope_scaling_factor: float | None
    local_rope_theta: float | None
    norm_eps: float
    tie_word_embeddings: bool
    # mixture of experts (num_experts == 0 means dense)
    moe_intermediate_size: int = 0
    num_experts: int = 0
    num_experts_per_tok: int = 0
    mlp_only_layers: tuple[int, ...] = ()
    decoder_sparse_step: int = 1
    norm_topk_prob: bool = True
    aux_loss_coef: float = 0.0
    shd_cfg: ShardConfig = dataclasses.field(default_factory=ShardConfig.default)
    dtype: Any = torch.bfloat16

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def variant(self) -> str:
        return "moe" if self.is_moe else "dense"

    def is_moe_layer(self, layer_idx: int) -> bool:
        return (
            self.is_moe
            and layer_idx not in self.mlp_only_layers
            and (layer_idx + 1) % self.decoder_sparse_step == 0
        )

    @classmethod
    def with_sharding(cls, **kw):
        kw.pop("variant", None)
        kw["shd_cfg"] = ShardConfig.default()
        return cls(**kw)


_BASE = dict(rope_theta=1_000_000, rope_scaling_factor=None, local_rope_theta=None, norm_eps=1e-6,
             tie_word_embeddings=False)

_SMOKE_SPECS: dict[str, dict[str, Any]] = {
    "qwen3-smoke": dict(vocab_size=1024, emb_dim=128, mlp_dim=512, num_layers=2, num_heads=4,
                        head_dim=32, num_kv_heads=4, **_BASE),
    "qwen3-smoke-moe": dict(vocab_size=512, emb_dim=128, mlp_dim=256, moe_intermediate_size=256,
                            num_layers=2, num_heads=4, head_dim=32, num_kv_heads=4, num_experts=4,
                            num_experts_per_tok=2, mlp_only_layers=(), decoder_sparse_step=1,
                            norm_topk_prob=True, **_BASE),
    # the CPU fp32 acceptance configuration: 2 layers, hidden 64, 4 Q / 2 KV heads, head_dim 16,
    # SwiGLU 128, vocabulary 1024 with tied embeddings
    "qwen3-smoke-tiny": dict(vocab_size=1024, emb_dim=64, mlp_dim=128, num_layers=2, num_heads=4,
                             head_dim=16, num_kv_heads=2, **{**_BASE, "tie_word_embeddings": True}),
}

# Architecture presets for the published checkpoints, so that benchmarks and random-init runs
# work without a config.json on disk (values are those of the public HF configs).
_ARCH_SPECS: dict[str, dict[str, Any]] = {
    "Qwen/Qwen3-0.6B": dict(vocab_size=151936, emb_dim=1024, mlp_dim=3072, num_layers=28, num_heads=16,
                            head_dim=128, num_kv_heads=8, **{**_BASE, "tie_word_embeddings": True}),
    "Qwen/Qwen3-1.7B": dict(vocab_size=151936, emb_dim=2048, mlp_dim=6144, num_layers=28, num_heads=16,
                            head_dim=128, num_kv_heads=8, **{**_BASE, "tie_word_embeddings": True}),
    "Qwen/Qwen3-4B": dict(vocab_size=151936, emb_dim=2560, mlp_dim=9728, num_layers=36, num_heads=32,
                          head_dim=128, num_kv_heads=8, **{**_BASE, "tie_word_embeddings": True}),
    "Qwen/Qwen3-8B": dict(vocab_size=151936, emb_dim=4096, mlp_dim=12288, num_layers=36, num_heads=32,
                          head_dim=128, num_kv_heads=8, **_BASE),
    "Qwen/Qwen3-14B": dict(vocab_size=151936, emb_dim=5120, mlp_dim=17408, num_layers=40, num_heads=40,
                           head_dim=128, num_kv_heads=8, **_BASE),
    "Qwen/Qwen3-32B": dict(vocab_size=151936, emb_dim=5120, mlp_dim=25600, num_layers=64, num_heads=64,
                           head_dim=128, num_kv_heads=8, **_BASE),
    "Qwen/Qwen3-30B-A3B-Instruct-2507": dict(
        vocab_size=151936, emb_dim=2048, mlp_dim=6144, moe_intermediate_size=768, num_layers=48,
        num_heads=32, head_dim=128, num_kv_heads=4, num_experts=128, num_experts_per_tok=8,
        mlp_only_layers=(), decoder_sparse_step=1, norm_topk_prob=True, aux_loss_coef=0.001,
        **{**_BASE, "rope_theta": 10_000_000}),
}

_DENSE_REPOS = ("Qwen/Qwen3-0.6B", "Qwen/Qwen3-1.7B", "Qwen/Qwen3-4B", "Qwen/Qwen3-8B",
                "Qwen/Qwen3-14B", "Qwen/Qwen3-32B")
_MOE_REPOS = ("Qwen/Qwen3-30B-A3B-Instruct-2507",)
_REAL_MODEL_IDS = (*_DENSE_REPOS, *_MOE_REPOS)
_SUPPORTED_MODEL_IDS = sorted((*_SMOKE_SPECS, *_REAL_MODEL_IDS))
_SUPPORTED_MODEL_TYPES = {"qwen3", "qwen3_moe"}


def list_qwen3_dense_model_ids() -> list[str]:
    return list(_DENSE_REPOS)


def list_qwen3_moe_model_ids() -> list[str]:
    return list(_MOE_REPOS)


def resolve_qwen3_repo_id(model_id: str) -> str:
    return model_id


def is_supported_model_id(model_id: str) -> bool:
    return model_id in _SMOKE_SPECS or model_id in _REAL_MODEL_IDS


def get_spec(model_id: str) -> dict[str, Any]:
    if model_id in _SMOKE_SPECS:
        return dict(_SMOKE_SPECS[model_id])
    if model_id in _REAL_MODEL_IDS:
        return {"hf_repo_id": model_id}
    raise ValueError(f"Unsupported Qwen3 model_id '{model_id}'. Supported ids: {_SUPPORTED_MODEL_IDS}")


def _required(m: dict, key: str, where: str):
    if key not in m:
        raise ValueError(f"Missing required key '{key}' in {where}.")
    return m[key]


def _required_any(m: dict, keys: tuple[str, ...], where: str):
    for k in keys:
        if k in m:
            return m[k]
    raise ValueError(f"Missing required key {' or '.join(repr(k) for k in keys)} in {where}.")


def make_config_from_hf(hf_cfg: dict[str, Any]) -> Qwen3Config:
    """Build a config from a HuggingFace ``config.json`` dict.  Accepts the transformers-5
    ``rope_parameters`` block or the legacy top-level ``rope_theta``."""
    model_type = _required(hf_cfg, "model_type", "hf_cfg")
    if model_type not in _SUPPORTED_MODEL_TYPES:
        raise ValueError(f"Unsupported Qwen3 model_type '{model_type}'. "
                         f"Expected one of {sorted(_SUPPORTED_MODEL_TYPES)}.")
    rp = hf_cfg.get("rope_parameters")
    if rp is None:
        rope_theta = _required(hf_cfg, "rope_theta", "hf_cfg")
        factor = local_theta = None
    else:
        if not isinstance(rp, dict):
            raise ValueError("Expected rope_parameters to be a dict in hf_cfg.")
        rope_theta = _required(rp, "rope_theta", "hf_cfg['rope_parameters']")
        if rp.get("rope_type", "default") != "default":
            raise ValueError(f"Unsupported rope_parameters.rope_type '{rp.get('rope_type')}' for Qwen3.")
        factor = rp.get("factor")
        local_theta = rp.get("local_rope_theta")
    moe = model_type == "qwen3_moe"
    return Qwen3Config(
        num_layers=_required(hf_cfg, "num_hidden_layers", "hf_cfg"),
        vocab_size=_required(hf_cfg, "vocab_size", "hf_cfg"),
        emb_dim=_required(hf_cfg, "hidden_size", "hf_cfg"),
        mlp_dim=_required(hf_cfg, "intermediate_size", "hf_cfg"),
        num_heads=_required(hf_cfg, "num_attention_heads", "hf_cfg"),
        head_dim=_required(hf_cfg, "head_dim", "hf_cfg"),
        num_kv_heads=_required(hf_cfg, "num_key_value_heads", "hf_cfg"),
        rope_theta=rope_theta,
        rope_scaling_factor=factor,
        local_rope_theta=local_theta,
        norm_eps=_required(hf_cfg, "rms_norm_eps", "hf_cfg"),
        tie_word_embeddings=_required(hf_cfg, "tie_word_embeddings", "hf_cfg"),
        moe_intermediate_size=_required(hf_cfg, "moe_intermediate_size", "hf_cfg") if moe else 0,
        num_experts=_required_any(hf_cfg, ("num_experts", "num_local_experts"), "hf_cfg") if moe
        else int(hf_cfg.get("num_experts", hf_cfg.get("num_local_experts", 0))),
        num_experts_per_tok=_required(hf_cfg, "num_experts_per_tok", "hf_cfg") if moe else 0,
        mlp_only_layers=tuple(_required(hf_cfg, "mlp_only_layers", "hf_cfg")) if moe else (),
        decoder_sparse_step=_required(hf_cfg, "decoder_sparse_step", "hf_cfg") if moe else 1,
        norm_topk_prob=_required(hf_cfg, "norm_topk_prob", "hf_cfg") if moe else True,
        aux_loss_coef=float(hf_cfg.get("router_aux_loss_coef", 0.0)),
        dtype=hf_dtype_to_torch(hf_cfg.get("dtype", hf_cfg.get("torch_dtype"))),
        shd_cfg=ShardConfig.default(),
    )


def make_config(model_id: str) -> Qwen3Config:
    """Smoke preset, local model directory, or repo id.  A repo id resolves through its
    ``config.json`` when one can be found and otherwise through the built-in architecture
    preset of that checkpoint."""
    if model_id in _SMOKE_SPECS:
        return Qwen3Config.with_sharding(**_SMOKE_SPECS[model_id])
    if "/" not in model_id and not Path(model_id).expanduser().exists():
        raise ValueError(f"Unsupported Qwen3 model_id '{model_id}'. Supported ids: {_SUPPORTED_MODEL_IDS}")
    try:
        return make_config_from_hf(load_hf_config_from_source(resolve_qwen3_repo_id(model_id)))
    except (ValueError, FileNotFoundError):
        if model_id in _ARCH_SPECS:
            return Qwen3Config.with_sharding(**_ARCH_SPECS[model_id])
        raise
