"""Export any supported model to the HuggingFace format (reference: omegalax/export.py)."""
from __future__ import annotations


def _family(obj_cfg):
    name = type(obj_cfg).__name__
    if name == "Qwen3Config":
        from .models.qwen3 import params as p

        return p.qwen3_to_hf_config_dict, p.export_qwen3_to_safetensors
    if name in ("Qwen3_5Config", "Qwen3_5TextConfig"):
        from .models.qwen3_5 import params as p

        return p.qwen3_5_to_hf_config_dict, p.export_qwen3_5_to_safetensors
    if name == "Qwen3VLConfig":
        from .models.qwen3_vl import params as p

        return p.qwen3_vl_to_hf_config_dict, p.export_qwen3_vl_to_safetensors
    raise TypeError(f"Unsupported config type for export: {type(obj_cfg)}")


def export_model_to_hf(model, cfg, out_dir):
    """Write ``model.safetensors`` + ``config.json`` for ``model`` into ``out_dir``."""
    return _family(cfg)[1](model, cfg, out_dir)


def model_config_to_hf_dict(cfg) -> dict:
    return _family(cfg)[0](cfg)
