"""Load HuggingFace Qwen3.5 / Qwen3.5-MoE checkpoints (reference: omegalax/models/qwen3_5/loader.py).

Native fusions: q(+gate)/k/v -> ``attn.qkv_proj``; gate/up -> ``mlp.gate_up_proj``; experts are
already fused in HF (gate_up_proj [E,2F,D], down_proj [E,D,F]).  The Conv3d patch embedding
(O,C,T,H,W) is flattened to (O, C*T*H*W); the depthwise conv1d weight (C,1,K) to (C,K).
"""
from __future__ import annotations

import re

import torch

from ...parallel.mesh import ensure_mesh
from ..params_utils import (Rule, StateAssembler, Transform, load_hf_config, moe_rules, native_state, rows,
                            stream_safetensors)
from .config import Qwen3_5Config, make_config_from_hf
from .model import Qwen3_5ForConditionalGeneration


def vision_rules(prefix: str = r"model\.visual", native: str = "visual", deepstack: bool = False) -> list[Rule]:
    B = prefix + r"\.blocks\.(?P<b>\d+)"
    nb = lambda m: f"{native}.blocks.{m['b']}"  # noqa: E731
    rules = [
        Rule(prefix + r"\.patch_embed\.proj\.weight", lambda m: f"{native}.patch_embed.weight", transform=Transform.FLATTEN_OUT),
        Rule(prefix + r"\.patch_embed\.proj\.bias", lambda m: f"{native}.patch_embed.bias"),
        Rule(prefix + r"\.pos_embed\.weight", lambda m: f"{native}.pos_embed"),
    ]
    for hf, nat in (("norm1", "norm1"), ("norm2", "norm2"), ("attn.qkv", "attn.qkv"), ("attn.proj", "attn.proj"),
                    ("mlp.linear_fc1", "mlp.linear_fc1"), ("mlp.linear_fc2", "mlp.linear_fc2")):
        for wb in ("weight", "bias"):
            rules.append(Rule(B + r"\." + hf.replace(".", r"\.") + r"\." + wb,
                              (lambda nat, wb: lambda m: f"{nb(m)}.{nat}.{wb}")(nat, wb)))
    for part in ("norm", "linear_fc1", "linear_fc2"):
        for wb in ("weight", "bias"):
            rules.append(Rule(prefix + rf"\.merger\.{part}\.{wb}",
                              (lambda part, wb: lambda m: f"{native}.merger.{part}.{wb}")(part, wb)))
            if deepstack:
                rules.append(Rule(prefix + rf"\.deepstack_merger_list\.(?P<d>\d+)\.{part}\.{wb}",
                                  (lambda part, wb: lambda m: f"{native}.deepstack_mergers.{m['d']}.{part}.{wb}")(part, wb)))
    return rules


def text_rules(cfg, prefix: str = r"model\.language_model", native: str = "model") -> list[Rule]:
    H, G, K = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    L = prefix + r"\.layers\.(?P<l>\d+)"
    nl = lambda m: f"{native}.layers.{m['l']}"  # noqa: E731
    q_hi, k_hi, v_hi = 2 * H * K, (2 * H + G) * K, (2 * H + 2 * G) * K
    F = cfg.intermediate_size
    Fs = cfg.shared_expert_intermediate_size
    rules = [
        Rule(prefix + r"\.embed_tokens\.weight", lambda m: f"{native}.embedder.weight"),
        Rule(prefix + r"\.norm\.weight", lambda m: f"{native}.final_norm.weight"),
        Rule(r"lm_head\.weight", lambda m: "lm_head.weight"),
        Rule(L + r"\.input_layernorm\.weight", lambda m: nl(m) + ".input_norm.weight"),
        Rule(L + r"\.post_attention_layernorm\.weight", lambda m: nl(m) + ".post_norm.weight"),
        Rule(L + r"\.self_attn\.q_proj\.weight", lambda m: nl(m) + ".attn.qkv_proj.weight", lambda m: rows(0, q_hi)),
        Rule(L + r"\.self_attn\.k_proj\.weight", lambda m: nl(m) + ".attn.qkv_proj.weight", lambda m: rows(q_hi, k_hi)),
        Rule(L + r"\.self_attn\.v_proj\.weight", lambda m: nl(m) + ".attn.qkv_proj.weight", lambda m: rows(k_hi, v_hi)),
        Rule(L + r"\.self_attn\.q_proj\.bias", lambda m: nl(m) + ".attn.qkv_proj.bias", lambda m: rows(0, q_hi)),
        Rule(L + r"\.self_attn\.k_proj\.bias", lambda m: nl(m) + ".attn.qkv_proj.bias", lambda m: rows(q_hi, k_hi)),
        Rule(L + r"\.self_attn\.v_proj\.bias", lambda m: nl(m) + ".attn.qkv_proj.bias", lambda m: rows(k_hi, v_hi)),
        Rule(L + r"\.self_attn\.o_proj\.weight", lambda m: nl(m) + ".attn.o_proj.weight"),
        Rule(L + r"\.self_attn\.o_proj\.bias", lambda m: nl(m) + ".attn.o_proj.bias"),
        Rule(L + r"\.self_attn\.q_norm\.weight", lambda m: nl(m) + ".attn.q_norm.weight"),
        Rule(L + r"\.self_attn\.k_norm\.weight", lambda m: nl(m) + ".attn.k_norm.weight"),
        Rule(L + r"\.linear_attn\.in_proj_qkv\.weight", lambda m: nl(m) + ".linear_attn.in_proj_qkv.weight"),
        Rule(L + r"\.linear_attn\.in_proj_z\.weight", lambda m: nl(m) + ".linear_attn.in_proj_z.weight"),
        Rule(L + r"\.linear_attn\.in_proj_b\.weight", lambda m: nl(m) + ".linear_attn.in_proj_b.weight"),
        Rule(L + r"\.linear_attn\.in_proj_a\.weight", lambda m: nl(m) + ".linear_attn.in_proj_a.weight"),
        Rule(L + r"\.linear_attn\.out_proj\.weight", lambda m: nl(m) + ".linear_attn.out_proj.weight"),
        Rule(L + r"\.linear_attn\.conv1d\.weight", lambda m: nl(m) + ".linear_attn.conv_weight", transform=Transform.SQUEEZE1),
        Rule(L + r"\.linear_attn\.dt_bias", lambda m: nl(m) + ".linear_attn.dt_bias"),
        Rule(L + r"\.linear_attn\.A_log", lambda m: nl(m) + ".linear_attn.A_log"),
        Rule(L + r"\.linear_attn\.norm\.weight", lambda m: nl(m) + ".linear_attn.norm.weight"),
    ]
    if cfg.is_moe:
        rules += moe_rules(L, nl, cfg.moe_intermediate_size)
        rules += [
            Rule(L + r"\.mlp\.shared_expert\.gate_proj\.weight", lambda m: nl(m) + ".mlp.shared_expert.gate_up_proj.weight", lambda m: rows(0, Fs)),
            Rule(L + r"\.mlp\.shared_expert\.up_proj\.weight", lambda m: nl(m) + ".mlp.shared_expert.gate_up_proj.weight", lambda m: rows(Fs, 2 * Fs)),
            Rule(L + r"\.mlp\.shared_expert\.down_proj\.weight", lambda m: nl(m) + ".mlp.shared_expert.down_proj.weight"),
            Rule(L + r"\.mlp\.shared_expert_gate\.weight", lambda m: nl(m) + ".mlp.shared_expert_gate.weight"),
        ]
    else:
        rules += [
            Rule(L + r"\.mlp\.gate_proj\.weight", lambda m: nl(m) + ".mlp.gate_up_proj.weight", lambda m: rows(0, F)),
            Rule(L + r"\.mlp\.up_proj\.weight", lambda m: nl(m) + ".mlp.gate_up_proj.weight", lambda m: rows(F, 2 * F)),
            Rule(L + r"\.mlp\.down_proj\.weight", lambda m: nl(m) + ".mlp.down_proj.weight"),
        ]
    return rules


_DUP_LM = re.compile(r"(language_model\.)+")


def normalize_key(key: str) -> str:
    """Canonical HF key.  Some transformers releases re-apply their checkpoint renaming on save
    and emit ``model.language_model.language_model.language_model.*`` and
    ``model.language_model.visual.*``; both are folded back here."""
    key = _DUP_LM.sub("language_model.", key)
    if key.startswith("model.language_model.visual."):
        key = "model.visual." + key[len("model.language_model.visual."):]
    return key


def load_into(model, cfg: Qwen3_5Config, file_dir) -> None:
    asm = StateAssembler(native_state(model), vision_rules() + text_rules(cfg.text_config))
    for key, tensor in stream_safetensors(file_dir):
        key = normalize_key(key)
        if key.startswith("mtp."):  # multi-token-prediction heads are not part of the model
            continue
        asm.assign(key, tensor)
    tied = cfg.text_config.tie_word_embeddings and asm.filled["lm_head.weight"] == 0
    asm.finish(allow_unfilled=["lm_head.weight"] if tied else [])
    if tied:
        with torch.no_grad():
            model.lm_head.weight.copy_(model.model.embedder.weight)


def create_qwen3_5_from_safetensors(file_dir, model_id: str = "", *, tp_size=None, fsdp_size=None, dp_size=None,
                                    device="cpu", dtype=torch.float32):
    """Returns (model, cfg) for a directory with config.json + *.safetensors."""
    ensure_mesh(tp_size=tp_size, fsdp_size=fsdp_size, dp_size=dp_size)
    cfg = make_config_from_hf(load_hf_config(file_dir))
    model = Qwen3_5ForConditionalGeneration(cfg, device=device, dtype=dtype)
    load_into(model, cfg, file_dir)
    return model, cfg
