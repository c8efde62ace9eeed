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


def gather_tp_model(model, cfg, tp_group=None):
    """The unsplit (tp = 1) model assembled from the tensor-parallel ranks' slices, on every rank
    of ``tp_group`` (collective; default: the current tensor-parallel context's group)."""
    import importlib

    import torch
    import torch.distributed as dist

    if tp_group is None:
        from .parallel import tp as tp_lib

        ctx = tp_lib.current()
        tp_group = ctx.group if ctx is not None else None
    if tp_group is None:
        raise ValueError("a tensor-parallel model can only be exported with its process group (one call per rank)")
    layout = importlib.import_module(getattr(model, "TP_LAYOUT", "omegalax_b200.models.qwen3.tp_layout"))
    tp = dist.get_world_size(tp_group)
    first = next(model.parameters())
    full = type(model)(cfg, device=first.device, dtype=first.dtype)
    dst = dict(full.named_parameters())
    with torch.no_grad():
        for n, p in model.named_parameters():
            parts = [torch.empty_like(p) for _ in range(tp)]
            dist.all_gather(parts, p.detach().contiguous(), group=tp_group)
            dst[n].copy_(layout.tp_unslice(n, [q.cpu() for q in parts], cfg).to(first.device))
    return full


def export_model_to_hf(model, cfg, out_dir, tp_group=None):
    """Write ``model.safetensors`` + ``config.json`` for ``model`` into ``out_dir``.  A
    tensor-parallel model is first re-assembled over its group: every rank of the group makes the
    call, the first one writes."""
    if getattr(model, "tp_size", 1) > 1:
        import torch.distributed as dist

        model = gather_tp_model(model, cfg, tp_group)
        if dist.get_rank() != 0:
            return None
    return _family(cfg)[1](model, cfg, out_dir)


def model_config_to_hf_dict(cfg) -> dict:
    return _family(cfg)[0](cfg)
