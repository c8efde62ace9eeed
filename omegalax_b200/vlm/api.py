"""Public API for vision-language models (Qwen3.5, Qwen3-VL); mirrors omegalax/vlm/api.py."""
from __future__ import annotations

import dataclasses

import torch

from ..models import sharding_runtime as _rt
from ..models.hf_io import load_hf_config_from_source
from ..models.qwen3_5.config import (Qwen3_5Config, is_supported_qwen3_5_model_id, list_supported_qwen3_5_model_ids,
                                     make_config as make_qwen3_5_config,
                                     make_config_from_hf as make_qwen3_5_config_from_hf)
from ..models.qwen3_5.model import Qwen3_5ForConditionalGeneration
from ..models.qwen3_vl.config import (Qwen3VLConfig, is_supported_qwen3_vl_model_id,
                                      list_supported_qwen3_vl_model_ids, make_vl_config, make_vl_config_from_hf)
from ..models.qwen3_vl.model import Qwen3VL
from ..models.shard_config import shard_config_for_mesh
from ..parallel.mesh import Mesh, ensure_mesh

VLMConfig = Qwen3_5Config | Qwen3VLConfig


def resolve_config(model_or_id):
    if not isinstance(model_or_id, str):
        return model_or_id
    if is_supported_qwen3_5_model_id(model_or_id):
        return make_qwen3_5_config(model_or_id)
    if is_supported_qwen3_vl_model_id(model_or_id):
        return make_vl_config(model_or_id)
    hf_cfg = load_hf_config_from_source(model_or_id)
    mt = hf_cfg.get("model_type")
    if mt in {"qwen3_5", "qwen3_5_moe"}:
        return make_qwen3_5_config_from_hf(hf_cfg)
    if mt in {"qwen3_vl", "qwen3_vl_moe"}:
        return make_vl_config_from_hf(hf_cfg)
    raise ValueError(f"Unsupported VLM model/config source '{model_or_id}'. Supported Qwen3.5 ids: "
                     f"{list_supported_qwen3_5_model_ids()}; supported Qwen3-VL ids: {list_supported_qwen3_vl_model_ids()}.")


def _shd(cfg):
    return cfg.text_config.shd_cfg if isinstance(cfg, Qwen3_5Config) else cfg.shd_cfg


def align_config_to_mesh(cfg, mesh: Mesh):
    new = shard_config_for_mesh(_shd(cfg), mesh.shape)
    if isinstance(cfg, Qwen3_5Config):
        return dataclasses.replace(cfg, text_config=dataclasses.replace(cfg.text_config, shd_cfg=new))
    if isinstance(cfg, Qwen3VLConfig):
        return dataclasses.replace(cfg, shd_cfg=new)
    raise TypeError(f"Unsupported VLM config type: {type(cfg)}")


def batch_partition_spec(cfg):
    return (_shd(cfg).act_btd[0], None)


def shard_batch(token_ids_BT, cfg, mesh=None, device=None):
    return _rt.shard_batch(token_ids_BT, _shd(cfg), mesh, device)


def shard_batch_dict(batch: dict, cfg, mesh=None, device=None) -> dict:
    return _rt.shard_batch_dict(batch, _shd(cfg), mesh, device)


def vocab_size(cfg) -> int:
    if isinstance(cfg, Qwen3_5Config):
        return int(cfg.text_config.vocab_size)
    if isinstance(cfg, Qwen3VLConfig):
        return int(cfg.vocab_size)
    raise TypeError(f"Unsupported VLM config type: {type(cfg)}")


def model_class_for(cfg):
    if isinstance(cfg, Qwen3_5Config):
        return Qwen3_5ForConditionalGeneration
    if isinstance(cfg, Qwen3VLConfig):
        return Qwen3VL
    raise ValueError(f"Unsupported VLM config type: {type(cfg)}")


def init_model(model_or_id, rng: int = 0, *, tp_size=None, fsdp_size=None, dp_size=None, device=None, dtype=None,
               meta: bool = False):
    cfg = resolve_config(model_or_id)
    mesh = ensure_mesh(tp_size=tp_size, fsdp_size=fsdp_size, dp_size=dp_size)
    cfg = align_config_to_mesh(cfg, mesh)
    if device is None:
        device = "cuda" if torch.cuda.is_available() else "cpu"
    if dtype is None:
        base = cfg.text_config.dtype if isinstance(cfg, Qwen3_5Config) else cfg.dtype
        dtype = base if torch.device(device).type == "cuda" else torch.float32
    model = _rt.init_model_sharded(model_class_for(cfg), cfg, int(rng), mesh, meta=meta, device=device, dtype=dtype)
    return model, cfg


def forward(model, token_ids_BT, pad_id: int, cfg, *, attention_mask_BT=None, pixel_values=None,
            image_grid_thw=None, vision_cu_seqlens=None, position_ids_ZBT=None, return_local_rows: bool = False):
    """Hidden states before lm_head and the aux loss.  ``return_local_rows`` (tensor
    parallelism): this rank's sequence-parallel rows instead of the gathered [B,T,D]."""
    if attention_mask_BT is None:
        attention_mask_BT = (token_ids_BT != pad_id).to(torch.int32)
    if isinstance(model, Qwen3_5ForConditionalGeneration):
        return model(token_ids_BT, attention_mask_BT.to(torch.int32), pixel_values=pixel_values,
                     image_grid_thw=image_grid_thw, position_ids_ZBT=position_ids_ZBT,
                     return_local_rows=return_local_rows)
    if isinstance(model, Qwen3VL):
        return model(token_ids_BT, attention_mask_BT, position_ids_ZBT=position_ids_ZBT, pixel_values=pixel_values,
                     image_grid_thw=image_grid_thw, vision_cu_seqlens=vision_cu_seqlens,
                     return_local_rows=return_local_rows)
    raise ValueError(f"Unsupported VLM model type: {type(model)}")


def load_pretrained(model_id: str, *, tp_size=None, fsdp_size=None, dp_size=None, device="cpu", dtype=torch.float32):
    """Load pretrained weights from a local directory or (when reachable) the HF hub."""
    import os

    from ..models.qwen3_5.loader import create_qwen3_5_from_safetensors
    from ..models.qwen3_vl.loader import create_qwen3_vl_from_safetensors

    if os.path.isdir(model_id):
        local_dir = model_id
    else:
        from huggingface_hub import snapshot_download

        local_dir = snapshot_download(model_id)
    cfg = resolve_config(local_dir)
    kw = dict(tp_size=tp_size, fsdp_size=fsdp_size, dp_size=dp_size, device=device, dtype=dtype)
    if isinstance(cfg, Qwen3VLConfig):
        return create_qwen3_vl_from_safetensors(local_dir, **kw)
    if isinstance(cfg, Qwen3_5Config):
        return create_qwen3_5_from_safetensors(local_dir, **kw)
    raise ValueError(f"Unsupported VLM config type for pretrained loading: {type(cfg)}")


def make_cache(*_a, **_k):
    """Vision-language models have no KV-cache decode path; kept for interface symmetry."""
    return None


def decode(*_a, **_k):
    raise NotImplementedError("decode is not implemented for vision-language models.")
