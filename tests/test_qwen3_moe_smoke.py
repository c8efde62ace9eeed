"""Qwen3-MoE: routed-expert execution matches the HuggingFace model, per-expert key layout is
accepted, export writes the fused expert layout."""
import tempfile

import pytest
import torch
from safetensors.torch import load_file, save_file

from omegalax_b200.models.qwen3.loader import create_qwen3_from_safetensors
from omegalax_b200.models.qwen3.params import export_qwen3_to_safetensors
from omegalax_b200.parallel import mesh as mesh_lib
from omegalax_b200.text import api as text_api


@pytest.fixture(autouse=True)
def _mesh():
    mesh_lib.set_default_mesh(None)
    yield
    mesh_lib.set_default_mesh(None)


def _hf(tmp):
    from transformers import Qwen3MoeConfig, Qwen3MoeForCausalLM

    cfg = Qwen3MoeConfig(vocab_size=512, hidden_size=128, intermediate_size=256, moe_intermediate_size=64,
                         num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                         num_experts=4, num_experts_per_tok=2, norm_topk_prob=True, mlp_only_layers=[],
                         decoder_sparse_step=1, rms_norm_eps=1e-6, tie_word_embeddings=False,
                         rope_parameters={"rope_type": "default", "rope_theta": 1e6}, router_aux_loss_coef=0.001,
                         max_position_embeddings=256)
    torch.manual_seed(0)
    m = Qwen3MoeForCausalLM(cfg).float().eval()
    m.save_pretrained(tmp, safe_serialization=True)
    return m


def test_logits_match_hf_and_per_expert_layout():
    with tempfile.TemporaryDirectory() as tmp:
        hf = _hf(tmp)
        ours = create_qwen3_from_safetensors(tmp, tp_size=1, fsdp_size=1, dp_size=1)
        tok = torch.randint(1, 512, (2, 40))
        hidden, aux = text_api.forward(ours, tok, 0, ours.cfg)
        with torch.no_grad():
            ref = hf(input_ids=tok).logits
        torch.testing.assert_close(ours.lm_head(hidden), ref, rtol=2e-4, atol=2e-4)
        assert float(aux) > 0
        # rewrite the checkpoint with per-expert keys; the loader must accept that layout too
        import glob
        f = glob.glob(tmp + "/*.safetensors")[0]
        t = load_file(f)
        out = {}
        for k, v in t.items():
            if k.endswith("mlp.experts.gate_up_proj"):
                p = k[: -len("gate_up_proj")]
                F = v.shape[1] // 2
                for e in range(v.shape[0]):
                    out[f"{p}{e}.gate_proj.weight"] = v[e, :F].contiguous()
                    out[f"{p}{e}.up_proj.weight"] = v[e, F:].contiguous()
            elif k.endswith("mlp.experts.down_proj"):
                p = k[: -len("down_proj")]
                for e in range(v.shape[0]):
                    out[f"{p}{e}.down_proj.weight"] = v[e].contiguous()
            else:
                out[k] = v
        save_file(out, f)
        mesh_lib.set_default_mesh(None)
        again = create_qwen3_from_safetensors(tmp, tp_size=1, fsdp_size=1, dp_size=1)
        for (n1, p1), (n2, p2) in zip(ours.named_parameters(), again.named_parameters()):
            assert torch.equal(p1, p2), n1


def test_export_uses_fused_expert_layout_and_roundtrips():
    model, cfg = text_api.init_model("qwen3-smoke-moe", 0, tp_size=1, fsdp_size=1, dp_size=1, device="cpu")
    with tempfile.TemporaryDirectory() as tmp:
        export_qwen3_to_safetensors(model, cfg, tmp)
        t = load_file(tmp + "/model.safetensors")
        E, F, D = cfg.num_experts, cfg.moe_intermediate_size, cfg.emb_dim
        assert t["model.layers.0.mlp.experts.gate_up_proj"].shape == (E, 2 * F, D)
        assert t["model.layers.0.mlp.experts.down_proj"].shape == (E, D, F)
        assert t["model.layers.0.mlp.gate.weight"].shape == (E, D)
        mesh_lib.set_default_mesh(None)
        back = create_qwen3_from_safetensors(tmp, tp_size=1, fsdp_size=1, dp_size=1)
        for (n1, p1), (n2, p2) in zip(model.named_parameters(), back.named_parameters()):
            assert torch.equal(p1, p2), n1


def test_unmapped_key_is_reported():
    model, cfg = text_api.init_model("qwen3-smoke", 0, tp_size=1, fsdp_size=1, dp_size=1, device="cpu")
    with tempfile.TemporaryDirectory() as tmp:
        export_qwen3_to_safetensors(model, cfg, tmp)
        t = load_file(tmp + "/model.safetensors")
        t["model.layers.0.bogus.weight"] = torch.zeros(1)
        t.pop("model.norm.weight")
        save_file(t, tmp + "/model.safetensors")
        mesh_lib.set_default_mesh(None)
        with pytest.raises(RuntimeError) as e:
            create_qwen3_from_safetensors(tmp, tp_size=1, fsdp_size=1, dp_size=1)
        assert "bogus" in str(e.value) and "final_norm" in str(e.value)
