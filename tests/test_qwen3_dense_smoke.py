"""Qwen3 dense: logits parity with the HuggingFace model built in-process, left-padded
batches, export/load round trip (pattern: reference tests/test_qwen3_dense_smoke.py)."""
import tempfile

import pytest
import torch

from omegalax_b200.models.qwen3.loader import create_qwen3_from_safetensors
from omegalax_b200.models.qwen3.params import export_qwen3_to_safetensors
from omegalax_b200.text import api as text_api
from omegalax_b200.parallel import mesh as mesh_lib


@pytest.fixture(autouse=True)
def _mesh():
    mesh_lib.set_default_mesh(None)
    yield
    mesh_lib.set_default_mesh(None)


def _hf_model(tmp, tie=False, dtype=torch.float32):
    from transformers import Qwen3Config as HFConfig, Qwen3ForCausalLM

    cfg = HFConfig(vocab_size=1024, hidden_size=128, intermediate_size=512, num_hidden_layers=2,
                   num_attention_heads=4, num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-6,
                   tie_word_embeddings=tie, rope_parameters={"rope_type": "default", "rope_theta": 1_000_000},
                   attention_bias=False, max_position_embeddings=512)
    torch.manual_seed(0)
    m = Qwen3ForCausalLM(cfg).to(dtype).eval()
    m.save_pretrained(tmp, safe_serialization=True)
    return m


@pytest.mark.parametrize("tie", [False, True])
def test_logits_match_hf_fp32(tie):
    with tempfile.TemporaryDirectory() as tmp:
        hf = _hf_model(tmp, tie)
        ours = create_qwen3_from_safetensors(tmp, tp_size=1, fsdp_size=1, dp_size=1)
        tok = torch.randint(1, 1024, (2, 24))
        hidden, _ = text_api.forward(ours, tok, 0, ours.cfg)
        logits = ours.lm_head(hidden)
        with torch.no_grad():
            ref = hf(input_ids=tok).logits
        torch.testing.assert_close(logits, ref, rtol=1e-4, atol=1e-4)


def test_left_padded_batch_matches_hf():
    with tempfile.TemporaryDirectory() as tmp:
        hf = _hf_model(tmp)
        ours = create_qwen3_from_safetensors(tmp, tp_size=1, fsdp_size=1, dp_size=1)
        tok = torch.randint(1, 1024, (3, 20))
        tok[0, :7] = 0
        tok[2, :3] = 0
        att = (tok != 0).long()
        hidden, _ = text_api.forward(ours, tok, 0, ours.cfg)
        logits = ours.lm_head(hidden)
        with torch.no_grad():
            ref = hf(input_ids=tok, attention_mask=att).logits
        m = att.bool()
        torch.testing.assert_close(logits[m], ref[m], rtol=1e-4, atol=1e-4)


def test_export_roundtrip_bit_equal():
    model, cfg = text_api.init_model("qwen3-smoke", 0, tp_size=1, fsdp_size=1, dp_size=1, device="cpu")
    with tempfile.TemporaryDirectory() as tmp:
        export_qwen3_to_safetensors(model, cfg, tmp)
        back = create_qwen3_from_safetensors(tmp, tp_size=1, fsdp_size=1, dp_size=1)
        for (n1, p1), (n2, p2) in zip(model.named_parameters(), back.named_parameters()):
            assert n1 == n2 and torch.equal(p1, p2), n1


def test_decode_matches_full_forward():
    model, cfg = text_api.init_model("qwen3-smoke-tiny", 0, tp_size=1, fsdp_size=1, dp_size=1, device="cpu")
    torch.manual_seed(0)
    tok = torch.randint(1, 1024, (2, 32))
    tok[1, :4] = 0  # left padding
    cache = text_api.make_cache(cfg, 2, 32, 8, dtype=torch.float32)
    logits, cache, _ = text_api.decode(model, cache, tok, 0, cfg)
    seq = tok
    for _ in range(8):
        nxt = logits[:, 1:].argmax(-1, keepdim=True) + 1  # never the pad id
        seq = torch.cat([seq, nxt], dim=1)
        logits, cache, _ = text_api.decode(model, cache, nxt, 0, cfg)
        with torch.no_grad():
            hidden, _ = text_api.forward(model, seq, 0, cfg)
            full = model.lm_head(hidden[:, -1])
        torch.testing.assert_close(logits, full, rtol=1e-4, atol=1e-4)
