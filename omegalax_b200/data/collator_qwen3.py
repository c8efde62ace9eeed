"""SFT collators for Qwen ChatML conversations (reference: omegalax/data/collator_qwen3.py).

Both return numpy dicts with ``token_ids_BT``, ``attention_mask_BT``, ``loss_mask_BT`` (int32,
``[B, max_length]``, right padded).  The loss mask is 1 on assistant content and on the
``<|im_end|>`` that closes it -- so the model learns to stop -- and 0 on the role header, the
newline after ``<|im_end|>`` and every non-assistant turn.
"""
from __future__ import annotations

from typing import Any, Sequence

import numpy as np

from .qwen3_encoding import encode_qwen_messages


def build_assistant_loss_mask(ids: np.ndarray, im_start_id: int, im_end_id: int, assistant_id: int) -> np.ndarray:
    """Vectorised: pair the k-th ``<|im_start|>`` with the k-th ``<|im_end|>``; for pairs whose
    header is ``assistant`` mark [start + 3, end] (header = start token, role token, newline)."""
    n = len(ids)
    mask = np.zeros(n + 1, dtype=np.int32)
    s = np.flatnonzero(ids == im_start_id)
    e = np.flatnonzero(ids == im_end_id)
    k = min(len(s), len(e))
    if k == 0:
        return mask[:n]
    s, e = s[:k], e[:k]
    sel = (s + 1 < n) & (ids[np.minimum(s + 1, n - 1)] == assistant_id)
    lo, hi = s[sel] + 3, e[sel] + 1
    ok = lo < n
    np.add.at(mask, lo[ok], 1)
    np.add.at(mask, np.minimum(hi[ok], n), -1)
    return np.cumsum(mask[:n]).astype(np.int32)


_build_assistant_loss_mask = build_assistant_loss_mask


class _Base:
    def __init__(self, tokenizer, max_length: int):
        if tokenizer.pad_token_id is None:
            raise ValueError("tokenizer must have pad_token_id set")
        self.tokenizer, self.max_length = tokenizer, max_length
        self._im_start = tokenizer.convert_tokens_to_ids("<|im_start|>")
        self._im_end = tokenizer.convert_tokens_to_ids("<|im_end|>")
        self._assistant = tokenizer.encode("assistant", add_special_tokens=False)[0]

    def _rows(self, ids: np.ndarray):
        n = len(ids)
        if n > self.max_length:
            raise ValueError(f"Encoded example length {n} exceeds max_length={self.max_length}; "
                             "rebuild the chunk index for this profile.")
        tok = np.full(self.max_length, self.tokenizer.pad_token_id, dtype=np.int32)
        att = np.zeros(self.max_length, dtype=np.int32)
        lm = np.zeros(self.max_length, dtype=np.int32)
        tok[:n] = ids
        att[:n] = 1
        lm[:n] = build_assistant_loss_mask(np.asarray(ids, dtype=np.int32), self._im_start, self._im_end, self._assistant)
        return tok, att, lm


class TextSFTCollator(_Base):
    def __call__(self, examples: Sequence[dict[str, Any]]) -> dict[str, np.ndarray]:
        rows = [self._rows(encode_qwen_messages(ex["messages"], tokenizer=self.tokenizer)["input_ids"]) for ex in examples]
        return {"token_ids_BT": np.stack([r[0] for r in rows]), "attention_mask_BT": np.stack([r[1] for r in rows]),
                "loss_mask_BT": np.stack([r[2] for r in rows])}


def compute_vision_cu_seqlens(image_grid_thw: np.ndarray) -> np.ndarray:
    """Cumulative per-frame token counts: every (t,h,w) contributes h*w, t times."""
    lens = []
    for t, h, w in np.asarray(image_grid_thw).tolist():
        lens += [int(h) * int(w)] * int(t)
    return np.concatenate([np.zeros(1, np.int32), np.cumsum(np.asarray(lens, dtype=np.int32), dtype=np.int32)])


_compute_vision_cu_seqlens = compute_vision_cu_seqlens


def pad_vision_arrays(pixel_values, image_grid_thw, merge_size: int, max_patches: int, max_images: int):
    """Pad to exactly ``max_patches`` patch rows and ``max_images`` grid rows with zero-pixel
    dummy images: ``n-1`` grids of (1, m, m) and one absorber (1, m, w*) sized to hit the patch
    budget, so device shapes are the same for every batch."""
    real_i, real_p = image_grid_thw.shape[0], pixel_values.shape[0]
    ms2 = merge_size * merge_size
    nd, extra = max_images - real_i, max_patches - real_p
    if nd < 0 or extra < 0:
        raise ValueError(f"Batch exceeds padding budget: real_images={real_i} > max_images={max_images} or "
                         f"real_patches={real_p} > max_patches={max_patches}. Increase the per-sample limits.")
    if nd == 0 and extra == 0:
        return pixel_values, image_grid_thw, compute_vision_cu_seqlens(image_grid_thw)
    if nd == 0 or extra < nd * ms2:
        raise ValueError(f"Vision budgets are infeasible for this batch: real_images={real_i}, real_patches={real_p}, "
                         f"max_images={max_images}, max_patches={max_patches}, ms2={ms2}. Padding needs at least one "
                         "dummy image and merge_size**2 patches per dummy; increase max_vision_images_per_sample or "
                         "max_vision_patches_per_sample.")
    absorber = extra - (nd - 1) * ms2
    if absorber % merge_size:
        raise ValueError(f"absorber_patches={absorber} not divisible by merge_size={merge_size}; max_patches and every "
                         "real image (h*w) must be multiples of merge_size.")
    dummies = [[1, merge_size, absorber // merge_size]] + [[1, merge_size, merge_size]] * (nd - 1)
    grid = np.concatenate([image_grid_thw, np.asarray(dummies, dtype=image_grid_thw.dtype)], 0)
    pv = np.concatenate([pixel_values, np.zeros((extra, pixel_values.shape[1]), pixel_values.dtype)], 0)
    return pv, grid, compute_vision_cu_seqlens(grid)


_pad_vision_arrays = pad_vision_arrays


class VLMSFTCollator(_Base):
    """Adds ``pixel_values`` [sum N, C*tp*p*p], ``image_grid_thw`` [M,3], ``vision_cu_seqlens`` and
    host-computed ``position_ids_ZBT`` [3,B,T] when the batch contains images."""

    def __init__(self, tokenizer, max_length: int, image_processor, *, max_vision_patches_per_sample: int | None = None,
                 max_vision_images_per_sample: int | None = None):
        super().__init__(tokenizer, max_length)
        self.image_processor = image_processor
        self._max_p, self._max_i = max_vision_patches_per_sample, max_vision_images_per_sample
        self._image_id = tokenizer.convert_tokens_to_ids("<|image_pad|>")
        self._video_id = tokenizer.convert_tokens_to_ids("<|video_pad|>")
        self._vstart_id = tokenizer.convert_tokens_to_ids("<|vision_start|>")

    def __call__(self, examples: Sequence[dict[str, Any]]) -> dict[str, np.ndarray]:
        from ..models.qwen3_vl.model import get_rope_index

        rows, pix, grids = [], [], []
        for ex in examples:
            enc = encode_qwen_messages(ex["messages"], tokenizer=self.tokenizer, image_processor=self.image_processor,
                                       include_pixels=True)
            rows.append(self._rows(enc["input_ids"]))
            if "pixel_values" in enc:
                pix.append(enc["pixel_values"])
                grids.append(enc["image_grid_thw"])
        out = {"token_ids_BT": np.stack([r[0] for r in rows]), "attention_mask_BT": np.stack([r[1] for r in rows]),
               "loss_mask_BT": np.stack([r[2] for r in rows])}
        if pix:
            pv, grid = np.concatenate(pix, 0), np.concatenate(grids, 0)
            merge = int(self.image_processor.merge_size)
            pos, _ = get_rope_index(out["token_ids_BT"], image_grid_thw=grid, attention_mask=out["attention_mask_BT"],
                                    spatial_merge_size=merge, image_token_id=self._image_id,
                                    video_token_id=self._video_id, vision_start_token_id=self._vstart_id)
            out["position_ids_ZBT"] = pos.astype(np.int32)
            if self._max_p is not None and self._max_i is not None:
                pv, grid, cu = pad_vision_arrays(pv, grid, merge, self._max_p * len(examples), self._max_i * len(examples))
            else:
                cu = compute_vision_cu_seqlens(grid)
            out["pixel_values"], out["image_grid_thw"], out["vision_cu_seqlens"] = pv, grid, cu
        return out
