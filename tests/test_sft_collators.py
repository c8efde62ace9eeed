"""Collator semantics: ChatML text, loss mask (assistant content + its <|im_end|>), padding,
overflow errors, image pad counts and static-shape vision padding."""
import numpy as np
import pytest

from omegalax_b200.data.collator_qwen3 import (TextSFTCollator, VLMSFTCollator, build_assistant_loss_mask,
                                               compute_vision_cu_seqlens, pad_vision_arrays)
from omegalax_b200.data.qwen3_encoding import build_chatml_text, encode_qwen_messages
from omegalax_b200.data.stub_tokenizer import SimpleImageProcessor, StubTokenizer

MSGS = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"},
        {"role": "assistant", "content": "hello there"}, {"role": "user", "content": "bye"},
        {"role": "assistant", "content": "ciao"}]


def test_chatml_text():
    assert build_chatml_text(MSGS[:2], [], 1) == "<|im_start|>system\nbe brief<|im_end|>\n<|im_start|>user\nhi<|im_end|>\n"


def test_loss_mask_covers_assistant_content_and_im_end_only():
    tok = StubTokenizer()
    col = TextSFTCollator(tok, 96)
    out = col([{"messages": MSGS}])
    ids, lm, att = out["token_ids_BT"][0], out["loss_mask_BT"][0], out["attention_mask_BT"][0]
    assert ids.dtype == np.int32 and ids.shape == (96,)
    text = tok.decode(ids[lm == 1])
    assert text == "hello there<|im_end|>ciao<|im_end|>"
    n = int(att.sum())
    assert (ids[n:] == tok.pad_token_id).all() and lm[n:].sum() == 0
    im_end = tok.convert_tokens_to_ids("<|im_end|>")
    nl = tok.convert_tokens_to_ids("\n")
    for p in np.flatnonzero((ids == im_end) & (lm == 1)):
        assert ids[p + 1] == nl and lm[p + 1] == 0


def test_mask_builder_edge_cases():
    assert build_assistant_loss_mask(np.array([5, 6, 7]), 1, 2, 9).sum() == 0
    ids = np.array([1, 9, 10, 20, 21, 2, 10, 1, 8, 10, 30, 2])
    assert build_assistant_loss_mask(ids, 1, 2, 9).tolist() == [0, 0, 0, 1, 1, 1, 0, 0, 0, 0, 0, 0]


def test_overflow_raises():
    with pytest.raises(ValueError):
        TextSFTCollator(StubTokenizer(), 8)([{"messages": MSGS}])


def _img_msgs(h=64, w=96):
    img = np.random.RandomState(0).rand(h, w, 3)
    return [{"role": "user", "content": [{"type": "image", "image": img}, {"type": "text", "text": "describe"}]},
            {"role": "assistant", "content": "a picture"}]


def test_image_pad_count_matches_grid():
    tok, ip = StubTokenizer(), SimpleImageProcessor(16, 2, 2)
    enc = encode_qwen_messages(_img_msgs(), tokenizer=tok, image_processor=ip, include_pixels=True)
    t, h, w = enc["image_grid_thw"][0]
    n_pad = int((enc["input_ids"] == tok.convert_tokens_to_ids("<|image_pad|>")).sum())
    assert n_pad == t * (h // 2) * (w // 2)
    assert enc["pixel_values"].shape == (t * h * w, 3 * 2 * 16 * 16)


def test_vlm_collator_outputs_and_static_padding():
    tok, ip = StubTokenizer(), SimpleImageProcessor(16, 2, 2)
    col = VLMSFTCollator(tok, 160, ip, max_vision_patches_per_sample=64, max_vision_images_per_sample=3)
    out = col([{"messages": _img_msgs()}, {"messages": _img_msgs(32, 32)}])
    assert out["pixel_values"].shape[0] == 128 and out["image_grid_thw"].shape == (6, 3)
    g = out["image_grid_thw"]
    assert int((g[:, 0] * g[:, 1] * g[:, 2]).sum()) == 128
    assert out["vision_cu_seqlens"][-1] == 128 and out["position_ids_ZBT"].shape == (3, 2, 160)
    assert np.array_equal(out["vision_cu_seqlens"], compute_vision_cu_seqlens(g))
    text_only = col([{"messages": MSGS}])
    assert "pixel_values" not in text_only


def test_pad_vision_arrays_errors():
    pv, grid = np.zeros((16, 4), np.float32), np.array([[1, 4, 4]])
    with pytest.raises(ValueError):
        pad_vision_arrays(pv, grid, 2, 8, 2)
    with pytest.raises(ValueError):
        pad_vision_arrays(pv, grid, 2, 18, 2)  # a dummy needs at least merge**2 patches
    out = pad_vision_arrays(pv, grid, 2, 16, 1)
    assert out[0] is pv
