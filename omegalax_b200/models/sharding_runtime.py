"""Born-sharded model construction and per-process batch placement.

``init_model_sharded`` builds the module tree on the meta device (no full replica is ever
allocated) and returns it together with the mesh; the training engine then materialises
only this rank's slice of every parameter.  ``shard_batch`` / ``shard_batch_dict`` move a
process-local batch (numpy or CPU tensors; dim 0 is this rank's share of the global batch)
onto the device through pinned host memory.
Reference: omegalax/models/sharding_runtime.py:14-76.
"""
from __future__ import annotations

import numpy as np
import torch

_ATTN_BACKEND = {"text": "sm100"}


def init_model_sharded(model_cls, cfg, seed: int, mesh, *, meta: bool = True, device=None, dtype=None):
    import inspect

    torch.manual_seed(int(seed))
    kw = {}
    tp = getattr(mesh, "tp", 1) if mesh is not None else 1
    if tp > 1:
        if "tp_size" not in inspect.signature(model_cls.__init__).parameters:
            raise NotImplementedError(f"{model_cls.__name__} has no tensor-parallel layout (tp_size={tp})")
        kw["tp_size"] = tp
    if meta:
        with torch.device("meta"):
            return model_cls(cfg, dtype=dtype or torch.float32, **kw)
    return model_cls(cfg, device=device, dtype=dtype or torch.float32, **kw)


def set_attn_backend(model, backend: str) -> None:
    """Select the text attention implementation: "sm100" (tcgen05 kernels) or "reference"
    (PyTorch definition).  Accepts the reference's backend names and maps every GPU kernel
    backend onto "sm100"."""
    name = {"mosaic_gpu": "sm100", "mosaic_tpu": "sm100", "cudnn": "sm100", "triton": "sm100",
            "xla": "reference"}.get(backend, backend)
    if name not in ("sm100", "reference"):
        raise ValueError(f"unknown attention backend '{backend}'")
    _ATTN_BACKEND["text"] = name
    setattr(model, "_attn_backend", name)


_PIN_CACHE: dict = {}


def _to_device(x, device, pinned: bool = True):
    if isinstance(x, np.ndarray):
        x = torch.from_numpy(np.ascontiguousarray(x))
    if not torch.is_tensor(x):
        return x
    dev = torch.device(device)
    if dev.type != "cuda":
        return x.to(dev)
    if pinned and not x.is_pinned():
        key = (tuple(x.shape), x.dtype)
        buf = _PIN_CACHE.get(key)
        if buf is None:
            buf = torch.empty(x.shape, dtype=x.dtype, pin_memory=True)
            _PIN_CACHE[key] = buf
        else:
            torch.cuda.current_stream().synchronize()  # previous copy out of this buffer is done
        buf.copy_(x)
        x = buf
    return x.to(dev, non_blocking=True)


def batch_partition_spec(shd_cfg):
    """Layout of a [B, T] batch: the batch dim over the data axes of the activation layout, the
    sequence dim whole (reference: omegalax/models/sharding_runtime.py:55-56)."""
    return (shd_cfg.act_btd[0], None)


def shard_batch(token_ids_BT, shd_cfg=None, mesh=None, device=None):
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    return _to_device(token_ids_BT, device)


_HOST_KEYS = ("image_grid_thw", "video_grid_thw")


def shard_batch_dict(batch: dict, shd_cfg=None, mesh=None, device=None) -> dict:
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    # image_grid_thw drives host-side loops (patch counts, position tables): it stays on the host,
    # reading it back from the device would stall the step on a synchronisation
    return {k: (_to_device(v, "cpu") if k in _HOST_KEYS else _to_device(v, device)) for k, v in batch.items()}
