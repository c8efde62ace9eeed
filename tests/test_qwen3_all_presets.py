"""Forward parity in fp32 for every registered Qwen3 checkpoint geometry.

The reference compares each published checkpoint with the HuggingFace model at rtol 1e-5 /
atol 1e-4 in fp32 (tests/test_qwen3_all_models.py:36-37,108).  The checkpoints cannot be fetched
here, so the same comparison runs on randomly initialised weights: every preset keeps its true
widths (hidden size, head count, KV head count, head dim, MLP width, expert count and width,
top-k, tied or untied head, rope theta) and is shortened to two layers (one for the
mixture-of-experts preset) and a 2048-entry vocabulary so that the seven models fit a CPU test.
The HuggingFace model is built from the configuration this package exports, saved as
safetensors and read back through the package's loader, so the config round trip, the key map
and the forward pass are all covered for each geometry.
"""
import dataclasses
import gc
import json
import os
import tempfile

import pytest
import torch

from omegalax_b200.models.qwen3 import config as qcfg
from omegalax_b200.models.qwen3.loader import create_qwen3_from_safetensors
from omegalax_b200.models.qwen3.params import qwen3_to_hf_config_dict
from omegalax_b200.parallel import mesh as mesh_lib
from omegalax_b200.text import api as text_api

RTOL, ATOL = 1e-5, 1e-4
_ALL = [*qcfg.list_qwen3_dense_model_ids(), *qcfg.list_qwen3_moe_model_ids()]


@pytest.fixture(autouse=True)
def _mesh():
    mesh_lib.set_default_mesh(None)
    yield
    mesh_lib.set_default_mesh(None)


@pytest.mark.parametrize("model_id", _ALL, ids=[m.split("/")[-1] for m in _ALL])
def test_prefill_logits_match_hf_fp32(model_id):
    import transformers as tf

    full = qcfg.make_config(model_id)
    cfg = dataclasses.replace(full, num_layers=1 if full.is_moe else 2, vocab_size=2048, dtype=torch.float32)
    hf_dict = qwen3_to_hf_config_dict(cfg)
    hf_dict["max_position_embeddings"] = 512
    hf_cls, hf_cfg_cls = ((tf.Qwen3MoeForCausalLM, tf.Qwen3MoeConfig) if cfg.is_moe
                          else (tf.Qwen3ForCausalLM, tf.Qwen3Config))
    hf_cfg = hf_cfg_cls(**{k: v for k, v in hf_dict.items() if k not in ("architectures", "model_type", "dtype")})
    torch.manual_seed(0)
    prev = torch.get_num_threads()
    with tempfile.TemporaryDirectory() as tmp:
        hf = hf_cls(hf_cfg).float().eval()
        # norm scales away from one and router logits away from zero, so that a swapped or skipped
        # norm / a wrong expert order cannot hide behind the default initialisation
        with torch.no_grad():
            for n, p in hf.named_parameters():
                if n.endswith("norm.weight"):
                    p.uniform_(0.5, 1.5)
        hf.save_pretrained(tmp, safe_serialization=True)
        assert json.load(open(os.path.join(tmp, "config.json")))["num_hidden_layers"] == cfg.num_layers
        ours = create_qwen3_from_safetensors(tmp, tp_size=1, fsdp_size=1, dp_size=1)
        for f in ("emb_dim", "mlp_dim", "num_heads", "num_kv_heads", "head_dim", "tie_word_embeddings", "rope_theta",
                  "num_experts", "num_experts_per_tok", "moe_intermediate_size", "norm_topk_prob"):
            assert getattr(ours.cfg, f) == getattr(full, f), f
        tok = torch.randint(1, cfg.vocab_size, (2, 19))
        tok[1, 15:] = 0                                   # right padding, as SFT batches have
        att = (tok != 0).long()
        hidden, _ = text_api.forward(ours, tok, 0, ours.cfg)
        logits = ours.lm_head(hidden)
        with torch.no_grad():
            ref = hf(input_ids=tok, attention_mask=att).logits
        m = att.bool()
        diff = (logits[m] - ref[m]).abs().max().item()
        torch.testing.assert_close(logits[m], ref[m], rtol=RTOL, atol=ATOL, msg=lambda s: f"{model_id}: {s} (max {diff:.3e})")
    del hf, ours
    gc.collect()
    torch.set_num_threads(prev)
