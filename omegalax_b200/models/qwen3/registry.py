"""Qwen3 family registry (reference: omegalax/models/qwen3/registry.py)."""
from __future__ import annotations

from .config import (Qwen3Config, is_supported_model_id, list_qwen3_dense_model_ids,
                     list_qwen3_moe_model_ids, make_config, make_config_from_hf)


def build_config(model_id: str) -> Qwen3Config:
    return make_config(model_id)


def get_model_cls(model_id: str | None = None):
    from .model import Qwen3

    return Qwen3


def infer_variant(model_id: str) -> str:
    return make_config(model_id).variant


__all__ = ["Qwen3Config", "build_config", "get_model_cls", "infer_variant", "is_supported_model_id",
           "list_qwen3_dense_model_ids", "list_qwen3_moe_model_ids", "make_config", "make_config_from_hf"]
