"""omegalax_b200: a Blackwell-native (sm_100a) LLM / VLM SFT and decode framework.

Public surface (mirrors omegalax/__init__.py): ``registry``, ``text_api``, ``vlm_api``,
``text_trainer``, ``vlm_trainer``, ``Cache``, ``LayerCache``, ``ShardConfig`` and the model
id listers.  Sub-packages are imported lazily so that importing the package is cheap.
"""
from __future__ import annotations

import importlib

__version__ = "0.1.0"

_LAZY = {
    "registry": "omegalax_b200.registry",
    "text_api": "omegalax_b200.text.api",
    "vlm_api": "omegalax_b200.vlm.api",
    "text_trainer": "omegalax_b200.trainers.text",
    "vlm_trainer": "omegalax_b200.trainers.vlm",
    "export": "omegalax_b200.export",
}
_ATTRS = {
    "Cache": ("omegalax_b200.models.qwen3.cache", "Cache"),
    "LayerCache": ("omegalax_b200.models.qwen3.cache", "LayerCache"),
    "ShardConfig": ("omegalax_b200.models.shard_config", "ShardConfig"),
    "Qwen3_5Config": ("omegalax_b200.models.qwen3_5.config", "Qwen3_5Config"),
    "Qwen3_5TextConfig": ("omegalax_b200.models.qwen3_5.config", "Qwen3_5TextConfig"),
    "Qwen3_5ForCausalLM": ("omegalax_b200.models.qwen3_5.model", "Qwen3_5ForCausalLM"),
    "Qwen3_5ForConditionalGeneration": ("omegalax_b200.models.qwen3_5.model", "Qwen3_5ForConditionalGeneration"),
    "list_qwen3_dense_model_ids": ("omegalax_b200.models.qwen3.config", "list_qwen3_dense_model_ids"),
    "list_qwen3_moe_model_ids": ("omegalax_b200.models.qwen3.config", "list_qwen3_moe_model_ids"),
}


def __getattr__(name):
    if name in _LAZY:
        return importlib.import_module(_LAZY[name])
    if name in _ATTRS:
        mod, attr = _ATTRS[name]
        return getattr(importlib.import_module(mod), attr)
    raise AttributeError(name)
