"""RoPE tables are generated in fp32 and applied in the model dtype for the text stacks; the
vision rotary is applied in fp32 and cast back."""
from unittest import mock

import torch

from omegalax_b200.models.qwen3 import rope as q3rope
from omegalax_b200.models.qwen3_5 import rope as q35rope
from omegalax_b200.models.qwen3_vl.model import compute_mrope_pos_embeddings
from omegalax_b200.ops import reference as R


def test_tables_are_fp32():
    pos = torch.arange(10)
    s, c = q3rope.generate_pos_embeddings(pos[None], 16)
    assert s.dtype == c.dtype == torch.float32 and s.shape == (1, 10, 8)
    p3 = pos[None, None].expand(3, 1, 10)
    c2, s2 = q35rope.generate_text_rope(p3, 32, 0.25, 1e4, (2, 1, 1))
    assert c2.dtype == torch.float32 and c2.shape == (1, 10, 8)
    s3, c3 = compute_mrope_pos_embeddings(p3, 32, 1e6, (8, 4, 4))
    assert s3.dtype == torch.float32 and s3.shape == (1, 10, 16)


def test_text_rope_applies_in_model_dtype():
    x = torch.randn(2, 5, 3, 16, dtype=torch.bfloat16)
    s, c = q3rope.generate_pos_embeddings(torch.arange(5)[None].expand(2, 5), 16)
    seen = {}
    real = R.apply_rope

    def spy(x, sin, cos, rot=None):
        out = real(x, sin, cos, rot)
        seen["out"] = out.dtype
        return out

    with mock.patch.object(R, "apply_rope", spy):
        y = q3rope.apply_rope(x, s, c)
    assert y.dtype == torch.bfloat16 and seen["out"] == torch.bfloat16
    # the multiplication happens with bf16 tables: identical to an explicit bf16 evaluation
    s16, c16 = s.to(torch.bfloat16).unsqueeze(-2), c.to(torch.bfloat16).unsqueeze(-2)
    x1, x2 = x[..., :8], x[..., 8:]
    assert torch.equal(y, torch.cat([x1 * c16 - x2 * s16, x2 * c16 + x1 * s16], -1))


def test_partial_rotary_passes_remaining_channels():
    x = torch.randn(1, 4, 2, 32)
    cos, sin = q35rope.generate_text_rope(torch.arange(4)[None, None].expand(3, 1, 4), 32, 0.25, 1e4, (2, 1, 1))
    y = q35rope.apply_text_rope(x, cos, sin)
    assert torch.equal(y[..., 8:], x[..., 8:]) and not torch.equal(y[..., :8], x[..., :8])


def test_vision_rope_runs_in_fp32_and_casts_back():
    x = torch.randn(6, 2, 8, dtype=torch.bfloat16)
    ang = torch.randn(6, 8)
    y = q35rope.apply_vision_rope(x, ang.cos(), ang.sin())
    xf = x.float()
    rot = torch.cat([-xf[..., 4:], xf[..., :4]], -1)
    want = (xf * ang.cos()[:, None] + rot * ang.sin()[:, None]).to(torch.bfloat16)
    assert y.dtype == torch.bfloat16 and torch.equal(y, want)


def test_mrope_interleave_rule():
    f = torch.stack([torch.full((1, 1, 8), float(a)) for a in (10, 20, 30)])
    out = q35rope.interleave_mrope(f, (4, 2, 2))[0, 0].tolist()
    assert out == [10, 20, 30, 10, 20, 30, 10, 10]
