"""Qwen3-VL (dense and MoE): text and image+text logits parity with HuggingFace models built
in-process, 3-D rope index parity, export/load round trip."""
import tempfile

import numpy as np
import pytest
import torch

from omegalax_b200.models.qwen3_vl import Qwen3VL, get_rope_index, make_vl_config
from omegalax_b200.models.qwen3_vl.loader import create_qwen3_vl_from_safetensors
from omegalax_b200.models.qwen3_vl.params import export_qwen3_vl_to_safetensors
from omegalax_b200.models.vision_common import vision_cu_seqlens
from omegalax_b200.parallel import mesh as mesh_lib

IMG, VID, VSTART = 1000, 1001, 1002


@pytest.fixture(autouse=True)
def _mesh():
    mesh_lib.set_default_mesh(None)
    yield
    mesh_lib.set_default_mesh(None)


def _hf(tmp, moe: bool):
    import transformers as tf

    text = dict(vocab_size=1024, hidden_size=128, intermediate_size=256, num_hidden_layers=3, num_attention_heads=4,
                num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-6,
                rope_parameters={"rope_type": "default", "rope_theta": 1e6, "mrope_section": [8, 4, 4], "mrope_interleaved": True},
                attention_bias=False, dtype="float32", max_position_embeddings=512)
    if moe:
        text.update(moe_intermediate_size=64, num_experts=4, num_experts_per_tok=2, mlp_only_layers=[],
                    decoder_sparse_step=1, norm_topk_prob=True)
    vision = dict(depth=3, hidden_size=64, intermediate_size=128, num_heads=4, patch_size=14, temporal_patch_size=2,
                  spatial_merge_size=2, in_channels=3, out_hidden_size=128, num_position_embeddings=256,
                  hidden_act="gelu_pytorch_tanh", deepstack_visual_indexes=[0, 1])
    kw = dict(text_config=text, vision_config=vision, tie_word_embeddings=False, image_token_id=IMG,
              video_token_id=VID, vision_start_token_id=VSTART, vision_end_token_id=1003)
    if moe:
        cfg, cls = tf.Qwen3VLMoeConfig(**kw), tf.Qwen3VLMoeForConditionalGeneration
    else:
        cfg, cls = tf.Qwen3VLConfig(**kw), tf.Qwen3VLForConditionalGeneration
    torch.manual_seed(0)
    m = cls(cfg).float().eval()
    m.save_pretrained(tmp, safe_serialization=True)
    return m


def _inputs():
    grid = [(1, 4, 6), (1, 4, 4)]
    n_merged = [t * (h // 2) * (w // 2) for t, h, w in grid]
    toks = [7, 8, VSTART] + [IMG] * n_merged[0] + [1003, 9, 10, VSTART] + [IMG] * n_merged[1] + [1003, 11, 12, 13]
    tok = torch.tensor([toks])
    torch.manual_seed(3)
    pix = torch.randn(sum(t * h * w for t, h, w in grid), 3 * 2 * 14 * 14)
    return tok, pix, grid


@pytest.mark.parametrize("moe", [False, True])
def test_text_and_image_logits_match_hf(moe):
    with tempfile.TemporaryDirectory() as tmp:
        hf = _hf(tmp, moe)
        ours, cfg = create_qwen3_vl_from_safetensors(tmp, tp_size=1, fsdp_size=1, dp_size=1)
        tok = torch.randint(5, 999, (2, 33))
        hidden, _ = ours(tok, torch.ones_like(tok))
        with torch.no_grad():
            ref = hf(input_ids=tok).logits
        torch.testing.assert_close(ours.lm_head(hidden), ref, rtol=2e-4, atol=2e-4)
        tok, pix, grid = _inputs()
        pos, _ = get_rope_index(tok.numpy(), grid, None, None, 2, IMG, VID, VSTART)
        hidden, _ = ours(tok, torch.ones_like(tok), torch.from_numpy(pos), pix, grid, vision_cu_seqlens(grid))
        with torch.no_grad():
            ref = hf(input_ids=tok, pixel_values=pix, image_grid_thw=torch.tensor(grid),
                     mm_token_type_ids=(tok == IMG).int()).logits
        torch.testing.assert_close(ours.lm_head(hidden), ref, rtol=3e-4, atol=3e-4)


def test_rope_index_matches_hf():
    with tempfile.TemporaryDirectory() as tmp:
        hf = _hf(tmp, False)
        tok, pix, grid = _inputs()
        tok2 = torch.cat([tok, tok], 0)
        att = torch.ones_like(tok2)
        att[1, :3] = 0
        tok2[1, :3] = 0
        # second row: shift so that its vision spans stay intact after left padding
        row = tok[0].tolist()
        tok2[1] = torch.tensor([0, 0, 0] + row[:-3])
        ours, deltas = get_rope_index(tok2.numpy(), grid + grid, None, att.numpy(), 2, IMG, VID, VSTART)
        ref, ref_d = hf.model.get_rope_index(tok2, (tok2 == IMG).int(), image_grid_thw=torch.tensor(grid + grid),
                                             attention_mask=att)
        m = att.bool()
        assert np.array_equal(ours[:, m.numpy()], ref[:, m].numpy())


@pytest.mark.parametrize("mid", ["qwen3-vl-smoke", "qwen3-vl-smoke-moe"])
def test_export_roundtrip(mid):
    cfg = make_vl_config(mid)
    torch.manual_seed(2)
    model = Qwen3VL(cfg)
    with tempfile.TemporaryDirectory() as tmp:
        export_qwen3_vl_to_safetensors(model, cfg, tmp)
        back, cfg2 = create_qwen3_vl_from_safetensors(tmp, tp_size=1, fsdp_size=1, dp_size=1)
        assert cfg2.mrope_section == cfg.mrope_section
        for (n1, p1), (n2, p2) in zip(model.named_parameters(), back.named_parameters()):
            assert n1 == n2 and torch.equal(p1, p2), n1
