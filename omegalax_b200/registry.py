"""Model id -> architecture routing (reference: omegalax/registry.py).

Smoke aliases are classified by prefix; everything else by the ``model_type`` of its HF
config (``qwen3``/``qwen3_moe`` -> text; ``qwen3_5``/``qwen3_5_moe``/``qwen3_vl``/
``qwen3_vl_moe`` -> VLM), falling back to the built-in table of published checkpoints when
no config.json can be reached.
"""
from __future__ import annotations

from enum import Enum

from .models.hf_io import load_hf_config_from_source
from .models.qwen3.config import is_supported_model_id as _is_q3, resolve_qwen3_repo_id
from .models.qwen3_5.config import is_supported_qwen3_5_model_id as _is_q35, resolve_qwen3_5_repo_id
from .models.qwen3_vl.config import is_supported_qwen3_vl_model_id as _is_vl, resolve_qwen3_vl_repo_id


class Arch(str, Enum):
    TEXT = "text"
    VLM = "vlm"


_TEXT_MODEL_TYPES = {"qwen3", "qwen3_moe"}
_VLM_MODEL_TYPES = {"qwen3_5", "qwen3_5_moe", "qwen3_vl", "qwen3_vl_moe"}


def infer_arch(model_id: str) -> Arch:
    if model_id.startswith("qwen3-smoke"):
        return Arch.TEXT
    if model_id.startswith(("qwen3.5-smoke", "qwen3-vl-smoke", "qwen3.5-")):
        return Arch.VLM
    try:
        mt = load_hf_config_from_source(resolve_hf_repo_id(model_id)).get("model_type")
    except (ValueError, FileNotFoundError):
        if _is_q3(model_id):
            return Arch.TEXT
        if _is_q35(model_id) or _is_vl(model_id):
            return Arch.VLM
        raise ValueError(f"Unsupported model id '{model_id}'")
    if mt in _TEXT_MODEL_TYPES:
        return Arch.TEXT
    if mt in _VLM_MODEL_TYPES:
        return Arch.VLM
    raise ValueError(f"Cannot infer architecture for model/config source '{model_id}'")


def resolve_hf_repo_id(model_id: str) -> str:
    if "/" in model_id:
        return model_id
    if _is_q3(model_id):
        return resolve_qwen3_repo_id(model_id)
    if _is_q35(model_id):
        return resolve_qwen3_5_repo_id(model_id)
    if _is_vl(model_id):
        return resolve_qwen3_vl_repo_id(model_id)
    return model_id


def resolve(model_id: str) -> Arch:
    return infer_arch(model_id)
