"""Logit comparison thresholds for bf16 parity (max-abs < 2.0, median-abs < 0.2, top-1 agreement
> 0.9; same bounds as the reference's tests/logits_assert.py:5-7)."""
import torch

MAX_ABS, MEDIAN_ABS, TOP1 = 2.0, 0.2, 0.9


def assert_logits_close(ours, theirs, mask=None, top1=TOP1):
    ours, theirs = ours.float(), theirs.float()
    if mask is not None:
        ours, theirs = ours[mask], theirs[mask]
    diff = (ours - theirs).abs()
    assert float(diff.max()) < MAX_ABS, f"max abs diff {float(diff.max())}"
    assert float(diff.median()) < MEDIAN_ABS, f"median abs diff {float(diff.median())}"
    agree = (ours.argmax(-1) == theirs.argmax(-1)).float().mean()
    assert float(agree) > top1, f"top-1 agreement {float(agree)}"
