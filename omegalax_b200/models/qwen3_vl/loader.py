"""Load HuggingFace Qwen3-VL / Qwen3-VL-MoE checkpoints (reference: omegalax/models/qwen3_vl/loader.py)."""
from __future__ import annotations

import torch

from ...parallel.mesh import ensure_mesh
from ..params_utils import StateAssembler, load_hf_config, native_state, stream_safetensors
from ..qwen3.loader import key_rules as qwen3_text_rules
from ..qwen3_5.loader import normalize_key, vision_rules
from .config import Qwen3VLConfig, make_vl_config_from_hf
from .model import Qwen3VL


def key_rules(cfg: Qwen3VLConfig):
    return vision_rules(r"model\.visual", "visual", deepstack=True) + qwen3_text_rules(cfg, r"model\.language_model")


def load_into(model: Qwen3VL, cfg: Qwen3VLConfig, file_dir) -> None:
    asm = StateAssembler(native_state(model), key_rules(cfg))
    for key, tensor in stream_safetensors(file_dir):
        asm.assign(normalize_key(key), tensor)
    tied = cfg.tie_word_embeddings and asm.filled["lm_head.weight"] == 0
    asm.finish(allow_unfilled=["lm_head.weight"] if tied else [])
    if tied:
        with torch.no_grad():
            model.lm_head.weight.copy_(model.embedder.weight)


def create_qwen3_vl_from_safetensors(file_dir, model_id: str = "", *, tp_size=None, fsdp_size=None, dp_size=None,
                                     device="cpu", dtype=torch.float32):
    """Returns (model, cfg)."""
    ensure_mesh(tp_size=tp_size, fsdp_size=fsdp_size, dp_size=dp_size)
    cfg = make_vl_config_from_hf(load_hf_config(file_dir))
    model = Qwen3VL(cfg, device=device, dtype=dtype)
    load_into(model, cfg, file_dir)
    return model, cfg
