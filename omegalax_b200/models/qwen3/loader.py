"""Load a HuggingFace Qwen3 / Qwen3-MoE checkpoint (reference: omegalax/models/qwen3/loader.py)."""
from __future__ import annotations

import torch

from ...parallel.mesh import ensure_mesh
from ..params_utils import Rule, StateAssembler, load_hf_config, moe_rules, native_state, rows, stream_safetensors
from .config import Qwen3Config, make_config, make_config_from_hf
from .model import Qwen3


def key_rules(cfg: Qwen3Config, prefix: str = "model", native_prefix: str = "") -> list[Rule]:
    """HF key -> native slice rules.  ``prefix`` is the HF module path of the decoder."""
    H, G, K, F = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.mlp_dim
    L = rf"{prefix}\.layers\.(?P<l>\d+)"
    nl = lambda m: f"{native_prefix}layers.{m['l']}"  # noqa: E731
    q_hi, k_hi, v_hi = H * K, (H + G) * K, (H + 2 * G) * K
    rules = [
        Rule(rf"{prefix}\.embed_tokens\.weight", lambda m: f"{native_prefix}embedder.weight"),
        Rule(L + r"\.self_attn\.q_proj\.weight", lambda m: nl(m) + ".attn.qkv_proj.weight", lambda m: rows(0, q_hi)),
        Rule(L + r"\.self_attn\.k_proj\.weight", lambda m: nl(m) + ".attn.qkv_proj.weight", lambda m: rows(q_hi, k_hi)),
        Rule(L + r"\.self_attn\.v_proj\.weight", lambda m: nl(m) + ".attn.qkv_proj.weight", lambda m: rows(k_hi, v_hi)),
        Rule(L + r"\.self_attn\.o_proj\.weight", lambda m: nl(m) + ".attn.o_proj.weight"),
        Rule(L + r"\.self_attn\.q_norm\.weight", lambda m: nl(m) + ".attn.q_norm.weight"),
        Rule(L + r"\.self_attn\.k_norm\.weight", lambda m: nl(m) + ".attn.k_norm.weight"),
        Rule(L + r"\.input_layernorm\.weight", lambda m: nl(m) + ".input_norm.weight"),
        Rule(L + r"\.post_attention_layernorm\.weight", lambda m: nl(m) + ".post_norm.weight"),
        Rule(L + r"\.mlp\.gate_proj\.weight", lambda m: nl(m) + ".mlp.gate_up_proj.weight", lambda m: rows(0, F)),
        Rule(L + r"\.mlp\.up_proj\.weight", lambda m: nl(m) + ".mlp.gate_up_proj.weight", lambda m: rows(F, 2 * F)),
        Rule(L + r"\.mlp\.down_proj\.weight", lambda m: nl(m) + ".mlp.down_proj.weight"),
        Rule(rf"{prefix}\.norm\.weight", lambda m: f"{native_prefix}final_norm.weight"),
        Rule(r"lm_head\.weight", lambda m: f"{native_prefix}lm_head.weight"),
    ]
    if cfg.is_moe:
        rules += moe_rules(L, nl, cfg.moe_intermediate_size)
    return rules


def _assert_config(cfg: Qwen3Config, model_id: str) -> None:
    if not model_id:
        return
    try:
        want = make_config(model_id)
    except ValueError:
        return
    for f in ("num_layers", "vocab_size", "emb_dim", "num_heads", "num_kv_heads", "head_dim", "tie_word_embeddings"):
        if getattr(want, f) != getattr(cfg, f):
            raise ValueError(f"config mismatch for {model_id}: {f} is {getattr(cfg, f)} on disk, expected {getattr(want, f)}")


def load_into(model: Qwen3, cfg: Qwen3Config, file_dir, *, prefix: str = "model") -> None:
    asm = StateAssembler(native_state(model), key_rules(cfg, prefix))
    for key, tensor in stream_safetensors(file_dir):
        asm.assign(key, tensor)
    allow = ["lm_head.weight"] if cfg.tie_word_embeddings and asm.filled["lm_head.weight"] == 0 else []
    asm.finish(allow_unfilled=allow)
    if allow:  # tied head: the head is a copy of the embedding table
        with torch.no_grad():
            model.lm_head.weight.copy_(model.embedder.weight)


def create_qwen3_from_safetensors(file_dir, model_id: str = "", *, tp_size: int | None = None,
                                  fsdp_size: int | None = None, dp_size: int | None = None,
                                  device="cpu", dtype=torch.float32) -> Qwen3:
    """Build a Qwen3 from ``config.json`` + ``*.safetensors`` in ``file_dir``.  Every HF key
    must map and every native parameter must be filled, otherwise a RuntimeError lists them."""
    ensure_mesh(tp_size=tp_size, fsdp_size=fsdp_size, dp_size=dp_size)
    cfg = make_config_from_hf(load_hf_config(file_dir))
    _assert_config(cfg, model_id)
    model = Qwen3(cfg, device=device, dtype=dtype)
    load_into(model, cfg, file_dir)
    return model
