"""HF config.json -> native config parsing, aliases, error cases, dtype defaults, registry."""
import pytest
import torch

from omegalax_b200 import registry
from omegalax_b200.export import model_config_to_hf_dict
from omegalax_b200.models.qwen3 import config as q3
from omegalax_b200.models.qwen3_5 import config as q35
from omegalax_b200.models.qwen3_vl import config as qvl

DENSE = {"model_type": "qwen3", "num_hidden_layers": 2, "vocab_size": 100, "hidden_size": 64, "intermediate_size": 128,
         "num_attention_heads": 4, "head_dim": 16, "num_key_value_heads": 2, "rms_norm_eps": 1e-6,
         "tie_word_embeddings": True, "rope_theta": 1e6}


def test_qwen3_dense_legacy_and_rope_parameters():
    c = q3.make_config_from_hf(DENSE)
    assert c.rope_theta == 1e6 and c.num_experts == 0 and not c.is_moe and c.dtype == torch.bfloat16
    d = dict(DENSE)
    d.pop("rope_theta")
    d["rope_parameters"] = {"rope_type": "default", "rope_theta": 5e5, "factor": 2.0}
    c = q3.make_config_from_hf(d)
    assert c.rope_theta == 5e5 and c.rope_scaling_factor == 2.0
    d["rope_parameters"]["rope_type"] = "yarn"
    with pytest.raises(ValueError):
        q3.make_config_from_hf(d)


def test_qwen3_moe_num_local_experts_alias_and_missing_keys():
    m = dict(DENSE, model_type="qwen3_moe", moe_intermediate_size=32, num_local_experts=8, num_experts_per_tok=2,
             mlp_only_layers=[0], decoder_sparse_step=1, norm_topk_prob=False, router_aux_loss_coef=0.01)
    c = q3.make_config_from_hf(m)
    assert c.num_experts == 8 and c.aux_loss_coef == 0.01 and not c.is_moe_layer(0) and c.is_moe_layer(1)
    m.pop("moe_intermediate_size")
    with pytest.raises(ValueError):
        q3.make_config_from_hf(m)
    with pytest.raises(ValueError):
        q3.make_config_from_hf({"model_type": "llama"})


def test_unknown_ids():
    with pytest.raises(ValueError):
        q3.make_config("qwen3-unknown")
    with pytest.raises(ValueError):
        q35.make_config("qwen3.5-unknown")
    with pytest.raises(ValueError):
        qvl.make_vl_config("qwen3-vl-unknown")
    assert q3.make_config("Qwen/Qwen3-8B").emb_dim == 4096  # built-in architecture table


def test_export_dict_roundtrip_all_families():
    for cfg in (q3.make_config("qwen3-smoke"), q3.make_config("qwen3-smoke-moe")):
        assert q3.make_config_from_hf(model_config_to_hf_dict(cfg)) == cfg
    for mid in ("qwen3.5-smoke", "qwen3.5-smoke-dense"):
        cfg = q35.make_config(mid)
        assert q35.make_config_from_hf(model_config_to_hf_dict(cfg)) == cfg
    for mid in ("qwen3-vl-smoke", "qwen3-vl-smoke-moe"):
        cfg = qvl.make_vl_config(mid)
        assert qvl.make_vl_config_from_hf(model_config_to_hf_dict(cfg)) == cfg


def test_vision_dtype_defaults_to_text_dtype():
    d = model_config_to_hf_dict(q35.make_config("qwen3.5-smoke"))
    d["text_config"]["dtype"] = "float32"
    d["vision_config"].pop("dtype")
    c = q35.make_config_from_hf(d)
    assert c.text_config.dtype == torch.float32 and c.vision_config.dtype == torch.float32
    d["vision_config"]["dtype"] = "bfloat16"
    assert q35.make_config_from_hf(d).vision_config.dtype == torch.bfloat16
    v = model_config_to_hf_dict(qvl.make_vl_config("qwen3-vl-smoke"))
    v["text_config"]["dtype"] = "float16"
    v["vision_config"].pop("dtype")
    assert qvl.make_vl_config_from_hf(v).vision.dtype == torch.float16


def test_qwen3_5_dense_xor_moe_and_vl_legacy_rope():
    d = model_config_to_hf_dict(q35.make_config("qwen3.5-smoke"))
    d["text_config"]["intermediate_size"] = 64
    with pytest.raises(ValueError):
        q35.make_config_from_hf(d)
    v = model_config_to_hf_dict(qvl.make_vl_config("qwen3-vl-smoke"))
    v["text_config"].pop("rope_parameters")  # legacy spelling only
    assert qvl.make_vl_config_from_hf(v).mrope_section == (8, 4, 4)


def test_registry_routing():
    assert registry.infer_arch("qwen3-smoke-moe") is registry.Arch.TEXT
    assert registry.infer_arch("qwen3-vl-smoke") is registry.Arch.VLM
    assert registry.resolve("Qwen/Qwen3-30B-A3B-Instruct-2507") is registry.Arch.TEXT
    assert registry.resolve_hf_repo_id("Qwen/Qwen3-8B") == "Qwen/Qwen3-8B"
