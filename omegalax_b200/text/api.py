"""Public API for text-only causal language models (Qwen3, Qwen3.5 text).

    model, cfg = init_model("qwen3-smoke", 0, tp_size=1, fsdp_size=1, dp_size=1)
    hidden, aux = forward(model, token_ids, pad_id, cfg)       # hidden is *before* lm_head
    cache = make_cache(cfg, batch, prompt_len, steps)
    logits, cache, aux = decode(model, cache, token_ids, pad_id, cfg)

Mirrors omegalax/text/api.py:42-146.
"""
from __future__ import annotations

import dataclasses

import torch

from ..models import sharding_runtime as _rt
from ..models.qwen3 import registry as qwen3_registry
from ..models.qwen3.cache import Cache, init_cache
from ..models.qwen3.model import Qwen3
from ..models.qwen3.paged_cache import PagedKVCache
from ..models.qwen3.utils import count_right_pads
from ..models.hf_io import load_hf_config_from_source
from ..models.shard_config import shard_config_for_mesh
from ..parallel.mesh import Mesh, ensure_mesh

ModelConfig = qwen3_registry.Qwen3Config
registry = qwen3_registry
list_qwen3_dense_model_ids = qwen3_registry.list_qwen3_dense_model_ids
list_qwen3_moe_model_ids = qwen3_registry.list_qwen3_moe_model_ids


def _q35():
    from ..models import qwen3_5

    return qwen3_5


def _is_q35_text(cfg) -> bool:
    return type(cfg).__name__ == "Qwen3_5TextConfig"


def resolve_config(model_or_id):
    """Model id (Qwen3 preset / repo, Qwen3.5 id -> its text config, or any directory / repo
    with a config.json) or an already-built config, which is passed through."""
    if not isinstance(model_or_id, str):
        return model_or_id
    if qwen3_registry.is_supported_model_id(model_or_id):
        return qwen3_registry.build_config(model_or_id)
    q35 = _q35()
    if q35.config.is_supported_qwen3_5_model_id(model_or_id):
        return q35.config.make_config(model_or_id).text_config
    hf_cfg = load_hf_config_from_source(model_or_id)
    mt = hf_cfg.get("model_type")
    if mt in {"qwen3", "qwen3_moe"}:
        return qwen3_registry.make_config_from_hf(hf_cfg)
    if mt in {"qwen3_5", "qwen3_5_moe"}:
        return q35.config.make_config_from_hf(hf_cfg).text_config
    raise ValueError(
        f"Unsupported text model/config source '{model_or_id}'. Supported Qwen3 ids: "
        f"{sorted(set(list_qwen3_dense_model_ids() + list_qwen3_moe_model_ids()))}; supported Qwen3.5 ids: "
        f"{q35.config.list_supported_qwen3_5_model_ids()}.")


def align_config_to_mesh(cfg, mesh: Mesh):
    """Drop size-one mesh axes from the config's activation layouts."""
    return dataclasses.replace(cfg, shd_cfg=shard_config_for_mesh(cfg.shd_cfg, mesh.shape))


def batch_partition_spec(cfg):
    return _rt.batch_partition_spec(cfg.shd_cfg)


def shard_batch(token_ids_BT, cfg, mesh: Mesh | None = None, device=None):
    return _rt.shard_batch(token_ids_BT, cfg.shd_cfg, mesh, device)


def shard_batch_dict(batch: dict, cfg, mesh: Mesh | None = None, device=None) -> dict:
    return _rt.shard_batch_dict(batch, cfg.shd_cfg, mesh, device)


def model_class_for(cfg):
    if isinstance(cfg, ModelConfig):
        return Qwen3
    if _is_q35_text(cfg):
        return _q35().model.Qwen3_5ForCausalLM
    raise ValueError(f"Unsupported text config type: {type(cfg)}")


def init_model(model_or_id, rng: int = 0, *, tp_size: int | None = None, fsdp_size: int | None = None,
               dp_size: int | None = None, device=None, dtype=None, meta: bool = False):
    """Random-initialise a text model; returns (model, cfg).  ``rng`` is an integer seed.
    With ``meta=True`` the parameters are not allocated (the training engine materialises
    only this rank's shard)."""
    cfg = resolve_config(model_or_id)
    mesh = ensure_mesh(tp_size=tp_size, fsdp_size=fsdp_size, dp_size=dp_size)
    cfg = align_config_to_mesh(cfg, mesh)
    if device is None:
        device = "cuda" if torch.cuda.is_available() else "cpu"
    if dtype is None:
        dtype = cfg.dtype if torch.device(device).type == "cuda" else torch.float32
    model = _rt.init_model_sharded(model_class_for(cfg), cfg, int(rng), mesh, meta=meta, device=device, dtype=dtype)
    return model, cfg


def forward(model, token_ids_BT, pad_id: int, cfg):
    """Hidden states before lm_head [B,T,D] and the auxiliary (router) loss."""
    segment_ids = (token_ids_BT != pad_id).to(torch.int32)
    return model(token_ids_BT, segment_ids, None, 0)


def decode(model, cache: Cache, token_ids_BT, pad_id: int, cfg):
    """One prefill / decode call: logits [B,V] at the last non-pad column, the cache, aux."""
    if not isinstance(model, Qwen3):
        raise NotImplementedError("decode is only implemented for Qwen3 text models.")
    segment_ids = (token_ids_BT != pad_id).to(torch.int32)
    if isinstance(cache, PagedKVCache):
        hidden = model.decode_paged(token_ids_BT, segment_ids, cache)
        with torch.no_grad():
            return model.lm_head(hidden), cache, torch.zeros((), device=hidden.device)
    nrp = count_right_pads(token_ids_BT, pad_id)
    with torch.no_grad():
        hidden, aux = model(token_ids_BT, segment_ids, cache, nrp)
        col = token_ids_BT.shape[-1] - nrp - 1
        logits = model.lm_head(hidden[:, col])
        if getattr(model, "vocab_parallel", False):   # this rank's slice of the vocabulary -> all of it
            from ..parallel import tp as tp_lib

            tp = tp_lib.current()
            parts = [torch.empty_like(logits) for _ in range(tp.size)]
            torch.distributed.all_gather(parts, logits.contiguous(), group=tp.group)
            logits = torch.cat(parts, dim=-1)
    return logits, cache, aux


def make_cache(cfg, batch_size: int, token_len: int, generate_steps: int, dtype=torch.bfloat16, device=None,
               paged: bool | None = None, page_size: int = 64, tp_size: int = 1):
    """KV cache for ``decode``.  On CUDA with bf16 (head_dim 128) the paged cache + decode kernels
    are used by default; otherwise the contiguous power-of-two cache of the reference.  With
    ``tp_size`` > 1 the (contiguous) cache holds this tensor-parallel rank's kv heads."""
    if not isinstance(cfg, ModelConfig):
        raise NotImplementedError("Cache is only available for Qwen3 text models.")
    if tp_size > 1:
        import dataclasses

        if cfg.num_kv_heads % tp_size:
            raise ValueError(f"kv heads ({cfg.num_kv_heads}) do not divide over tp_size={tp_size}")
        return init_cache(dataclasses.replace(cfg, num_kv_heads=cfg.num_kv_heads // tp_size), batch_size, token_len,
                          generate_steps, dtype, device)
    if paged is None:
        paged = (device is not None and torch.device(device).type == "cuda" and dtype == torch.bfloat16
                 and cfg.head_dim == 128 and (cfg.num_heads // cfg.num_kv_heads) in (1, 2, 4, 8))
    if paged:
        return PagedKVCache(cfg, batch_size, token_len + generate_steps, page_size=page_size, dtype=dtype, device=device)
    return init_cache(cfg, batch_size, token_len, generate_steps, dtype, device)
