"""Qwen3.5 (hybrid GatedDeltaNet / gated attention, dense and MoE): logits parity with the
HuggingFace model built in-process and export/load round trips."""
import tempfile

import pytest
import torch

from omegalax_b200.models.qwen3_5.config import make_config
from omegalax_b200.models.qwen3_5.loader import create_qwen3_5_from_safetensors
from omegalax_b200.models.qwen3_5.model import Qwen3_5ForConditionalGeneration
from omegalax_b200.models.qwen3_5.params import export_qwen3_5_to_safetensors
from omegalax_b200.parallel import mesh as mesh_lib


@pytest.fixture(autouse=True)
def _mesh():
    mesh_lib.set_default_mesh(None)
    yield
    mesh_lib.set_default_mesh(None)


def _hf(tmp, moe: bool):
    import transformers as tf

    text = dict(vocab_size=1024, hidden_size=128, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                head_dim=32, rms_norm_eps=1e-6, layer_types=["linear_attention"] * 3 + ["full_attention"],
                rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.25,
                                 "mrope_section": [2, 1, 1], "mrope_interleaved": True},
                linear_conv_kernel_dim=4, linear_key_head_dim=16, linear_num_key_heads=2, linear_num_value_heads=4,
                linear_value_head_dim=32, attention_bias=False, dtype="float32", max_position_embeddings=512)
    if moe:
        text.update(moe_intermediate_size=64, shared_expert_intermediate_size=64, num_experts=4, num_experts_per_tok=2,
                    router_aux_loss_coef=0.001)
    else:
        text.update(intermediate_size=256)
    vision = dict(depth=2, hidden_size=64, intermediate_size=128, num_heads=4, patch_size=16, temporal_patch_size=2,
                  spatial_merge_size=2, in_channels=3, out_hidden_size=128, num_position_embeddings=100)
    if moe:
        cfg = tf.Qwen3_5MoeConfig(text_config=text, vision_config=vision, tie_word_embeddings=False,
                                  image_token_id=1000, video_token_id=1001, vision_start_token_id=1002, vision_end_token_id=1003)
        cls = tf.Qwen3_5MoeForConditionalGeneration
    else:
        cfg = tf.Qwen3_5Config(text_config=text, vision_config=vision, tie_word_embeddings=False,
                               image_token_id=1000, video_token_id=1001, vision_start_token_id=1002, vision_end_token_id=1003)
        cls = tf.Qwen3_5ForConditionalGeneration
    torch.manual_seed(0)
    m = cls(cfg).float().eval()
    with torch.no_grad():  # make (1+w) norms and A_log / dt_bias non-trivial
        for n, p in m.named_parameters():
            if n.endswith("norm.weight") or "layernorm" in n:
                p.add_(0.1 * torch.randn_like(p))
    m.save_pretrained(tmp, safe_serialization=True)
    return m


@pytest.mark.parametrize("moe", [False, True])
def test_text_logits_match_hf(moe):
    with tempfile.TemporaryDirectory() as tmp:
        hf = _hf(tmp, moe)
        ours, cfg = create_qwen3_5_from_safetensors(tmp, tp_size=1, fsdp_size=1, dp_size=1)
        tok = torch.randint(1, 999, (2, 70))
        seg = torch.ones_like(tok)
        hidden, aux = ours(tok, seg)
        logits = ours.lm_head(hidden)
        with torch.no_grad():
            ref = hf(input_ids=tok).logits
        torch.testing.assert_close(logits, ref, rtol=2e-4, atol=2e-4)


@pytest.mark.parametrize("mid", ["qwen3.5-smoke", "qwen3.5-smoke-dense"])
def test_export_roundtrip(mid):
    cfg = make_config(mid)
    torch.manual_seed(1)
    model = Qwen3_5ForConditionalGeneration(cfg)
    with tempfile.TemporaryDirectory() as tmp:
        export_qwen3_5_to_safetensors(model, cfg, tmp)
        back, cfg2 = create_qwen3_5_from_safetensors(tmp, tp_size=1, fsdp_size=1, dp_size=1)
        assert cfg2.text_config.layer_types == cfg.text_config.layer_types
        for (n1, p1), (n2, p2) in zip(model.named_parameters(), back.named_parameters()):
            assert n1 == n2 and torch.equal(p1, p2), n1


@pytest.mark.parametrize("moe", [False, True])
def test_image_and_text_logits_match_hf(moe):
    """Pixels through the vision tower (patch embedding, interpolated position table, 2-D rotary
    attention, merger), spliced into the token sequence at the image placeholders, 3-D rotary
    positions from the grid: logits against ``Qwen3_5(Moe)ForConditionalGeneration``."""
    from omegalax_b200.models.qwen3_vl import get_rope_index

    IMG, VID, VSTART, VEND = 1000, 1001, 1002, 1003
    grid = [(1, 4, 6), (1, 6, 4)]
    n_merged = [t * (h // 2) * (w // 2) for t, h, w in grid]
    toks = [7, 8, VSTART] + [IMG] * n_merged[0] + [VEND, 9, 10, VSTART] + [IMG] * n_merged[1] + [VEND, 11, 12, 13]
    tok = torch.tensor([toks])
    torch.manual_seed(3)
    pix = torch.randn(sum(t * h * w for t, h, w in grid), 3 * 2 * 16 * 16)
    with tempfile.TemporaryDirectory() as tmp:
        hf = _hf(tmp, moe)
        ours, cfg = create_qwen3_5_from_safetensors(tmp, tp_size=1, fsdp_size=1, dp_size=1)
        pos, _ = get_rope_index(tok.numpy(), grid, None, None, 2, IMG, VID, VSTART)
        hidden, _ = ours(tok, torch.ones_like(tok), pix, grid, torch.from_numpy(pos))
        with torch.no_grad():
            ref = hf(input_ids=tok, pixel_values=pix, image_grid_thw=torch.tensor(grid),
                     mm_token_type_ids=(tok == IMG).int()).logits
        torch.testing.assert_close(ours.lm_head(hidden), ref, rtol=3e-4, atol=3e-4)
        # and the image must matter: without pixels the logits at the text tail differ
        hidden_txt, _ = ours(tok, torch.ones_like(tok))
        assert (ours.lm_head(hidden_txt)[0, -1] - ref[0, -1]).abs().max() > 1e-3
