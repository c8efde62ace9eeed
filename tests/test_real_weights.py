"""Parity against a checkpoint directory on local disk, for any of the three model families.

Opt-in for published checkpoints (no download is attempted):

    OMEGALAX_RUN_REAL_WEIGHTS_TESTS=1 OMEGALAX_REAL_WEIGHTS_DIR=/path/to/Qwen3-0.6B python -m pytest tests/test_real_weights.py

``OMEGALAX_REAL_WEIGHTS_DIR`` may hold several directories separated by ``:`` (e.g. a Qwen3, a
Qwen3.5 and a Qwen3-VL checkpoint).  For each: the family is taken from ``config.json``, the
loader must consume every tensor of the checkpoint and fill every parameter (it raises
otherwise), and the bf16 logits of a token batch are compared with the HuggingFace eager model (thresholds of the reference's
tests/logits_assert.py:5-7, top-1 agreement >= 0.8 as in tests/test_qwen3_0_6b.py:135,
tests/test_qwen3_5_0_8b.py and tests/test_qwen3_vl_2b.py).

The same routine always runs on three tiny checkpoints written by HuggingFace classes in a
temporary directory, so that the opt-in path itself is exercised on every run.
"""
import json
import os
import tempfile

import pytest
import torch

from tests.logits_assert import assert_logits_close

_DIRS = [d for d in os.environ.get("OMEGALAX_REAL_WEIGHTS_DIR", "").split(":") if d]
_ENABLED = bool(os.environ.get("OMEGALAX_RUN_REAL_WEIGHTS_TESTS")) and all(os.path.isdir(d) for d in _DIRS) and bool(_DIRS)


def check_checkpoint_dir(path: str, dtype=torch.bfloat16, top1: float = 0.8, batch=(2, 48)):
    """Load ``path`` with this package and with transformers; compare logits on random token ids."""
    import transformers as tf

    from omegalax_b200.parallel import mesh as mesh_lib
    from omegalax_b200.registry import Arch, infer_arch
    from omegalax_b200.text import api as text_api
    from omegalax_b200.vlm import api as vlm_api

    mesh_lib.set_default_mesh(None)
    try:
        hf_cfg = json.load(open(os.path.join(path, "config.json")))
        arch = infer_arch(path)
        if arch is Arch.TEXT:
            from omegalax_b200.models.qwen3.loader import create_qwen3_from_safetensors

            hf = tf.AutoModelForCausalLM.from_pretrained(path, torch_dtype=dtype).eval()
            ours = create_qwen3_from_safetensors(path, tp_size=1, fsdp_size=1, dp_size=1)
            cfg = ours.cfg
            vocab = cfg.vocab_size
        else:
            hf = tf.AutoModelForImageTextToText.from_pretrained(path, torch_dtype=dtype).eval()
            ours, cfg = vlm_api.load_pretrained(path, tp_size=1, fsdp_size=1, dp_size=1)
            vocab = vlm_api.vocab_size(cfg)
        assert arch is (Arch.TEXT if hf_cfg["model_type"] in ("qwen3", "qwen3_moe") else Arch.VLM)
        # (the loaders themselves raise when a checkpoint tensor matches no rule or a parameter stays unfilled)
        special = [hf_cfg.get(k) for k in ("image_token_id", "video_token_id", "vision_start_token_id", "vision_end_token_id")]
        hi = min([vocab, 32000] + [s for s in special if isinstance(s, int)])
        g = torch.Generator().manual_seed(0)
        tok = torch.randint(1, hi, batch, generator=g)
        ours = ours.to(dtype)
        with torch.no_grad():
            if arch is Arch.TEXT:
                hidden, _ = text_api.forward(ours, tok, 0, cfg)
            else:
                hidden, _ = vlm_api.forward(ours, tok, 0, cfg, attention_mask_BT=torch.ones_like(tok))
            logits = ours.lm_head(hidden)
            ref = hf(input_ids=tok).logits
        assert_logits_close(logits.float(), ref.float(), top1=top1)
    finally:
        mesh_lib.set_default_mesh(None)


@pytest.mark.skipif(not _ENABLED, reason="set OMEGALAX_RUN_REAL_WEIGHTS_TESTS=1 and OMEGALAX_REAL_WEIGHTS_DIR")
@pytest.mark.parametrize("path", _DIRS or ["-"])
def test_real_checkpoint_logits_match_hf(path):
    check_checkpoint_dir(path)


def _tiny(family: str, tmp: str):
    import transformers as tf

    torch.manual_seed(0)
    if family == "qwen3":
        cfg = tf.Qwen3Config(vocab_size=1024, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                             num_attention_heads=4, num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-6,
                             tie_word_embeddings=True, attention_bias=False, max_position_embeddings=256,
                             rope_parameters={"rope_type": "default", "rope_theta": 1_000_000})
        m = tf.Qwen3ForCausalLM(cfg)
    elif family == "qwen3_5":
        text = dict(vocab_size=1024, hidden_size=128, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                    head_dim=32, rms_norm_eps=1e-6, layer_types=["linear_attention"] * 3 + ["full_attention"],
                    rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.25,
                                     "mrope_section": [2, 1, 1], "mrope_interleaved": True},
                    linear_conv_kernel_dim=4, linear_key_head_dim=16, linear_num_key_heads=2, linear_num_value_heads=4,
                    linear_value_head_dim=32, attention_bias=False, dtype="float32", max_position_embeddings=256,
                    intermediate_size=256)
        vision = dict(depth=2, hidden_size=64, intermediate_size=128, num_heads=4, patch_size=16, temporal_patch_size=2,
                      spatial_merge_size=2, in_channels=3, out_hidden_size=128, num_position_embeddings=100)
        m = tf.Qwen3_5ForConditionalGeneration(tf.Qwen3_5Config(
            text_config=text, vision_config=vision, tie_word_embeddings=False, image_token_id=1000, video_token_id=1001,
            vision_start_token_id=1002, vision_end_token_id=1003))
    else:
        text = dict(vocab_size=1024, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-6, attention_bias=False, dtype="float32",
                    rope_parameters={"rope_type": "default", "rope_theta": 1e6, "mrope_section": [8, 4, 4],
                                     "mrope_interleaved": True}, max_position_embeddings=256)
        vision = dict(depth=2, hidden_size=64, intermediate_size=128, num_heads=4, patch_size=14, temporal_patch_size=2,
                      spatial_merge_size=2, in_channels=3, out_hidden_size=128, num_position_embeddings=256,
                      hidden_act="gelu_pytorch_tanh", deepstack_visual_indexes=[0, 1])
        m = tf.Qwen3VLForConditionalGeneration(tf.Qwen3VLConfig(
            text_config=text, vision_config=vision, tie_word_embeddings=False, image_token_id=1000, video_token_id=1001,
            vision_start_token_id=1002, vision_end_token_id=1003))
    m.float().eval().save_pretrained(tmp, safe_serialization=True)


@pytest.mark.parametrize("family", ["qwen3", "qwen3_5", "qwen3_vl"])
def test_checkpoint_directory_routine_on_tiny_models(family):
    """The opt-in routine, on a checkpoint directory that a HuggingFace class of each family wrote
    (fp32, so the bounds are met with a wide margin and top-1 agreement is near 1)."""
    with tempfile.TemporaryDirectory() as tmp:
        _tiny(family, tmp)
        check_checkpoint_dir(tmp, dtype=torch.float32, top1=0.95, batch=(2, 24))
