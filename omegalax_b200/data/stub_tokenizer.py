"""A dependency-free tokenizer with the Qwen ChatML special tokens and a byte fallback, for
tests, smoke runs and machines without a HuggingFace cache.  It exposes the small part of the
HF tokenizer surface that the collators use."""
from __future__ import annotations

import re

SPECIAL_TOKENS = ["<|endoftext|>", "<|im_start|>", "<|im_end|>", "<|vision_start|>", "<|vision_end|>",
                  "<|image_pad|>", "<|video_pad|>"]
_WORDS = ["system", "user", "assistant", "\n"]


class StubTokenizer:
    """ids: 0 pad/eos, 1..6 special tokens, then a few whole words ("assistant" is one token,
    as in the Qwen vocabulary), then 256 byte tokens."""

    def __init__(self):
        self.vocab = {t: i for i, t in enumerate(SPECIAL_TOKENS)}
        for w in _WORDS:
            self.vocab[w] = len(self.vocab)
        self.byte_base = len(self.vocab)
        self.pad_token_id = 0
        self.eos_token_id = 0
        self.vocab_size = self.byte_base + 256
        pats = [re.escape(t) for t in SPECIAL_TOKENS] + [r"\b(?:system|user|assistant)\b", "\n"]
        self._split = re.compile("(" + "|".join(pats) + ")")
        self._inv = {i: t for t, i in self.vocab.items()}

    def convert_tokens_to_ids(self, tok):
        if isinstance(tok, (list, tuple)):
            return [self.convert_tokens_to_ids(t) for t in tok]
        return self.vocab[tok]

    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        ids = []
        for piece in self._split.split(text):
            if not piece:
                continue
            if piece in self.vocab:
                ids.append(self.vocab[piece])
            else:
                ids.extend(self.byte_base + b for b in piece.encode("utf-8"))
        return ids

    def decode(self, ids) -> str:
        out, buf = [], bytearray()
        for i in ids:
            i = int(i)
            if i >= self.byte_base:
                buf.append(i - self.byte_base)
            else:
                if buf:
                    out.append(buf.decode("utf-8", errors="replace"))
                    buf = bytearray()
                out.append(self._inv.get(i, ""))
        if buf:
            out.append(buf.decode("utf-8", errors="replace"))
        return "".join(out)

    def __len__(self):
        return self.vocab_size


class SimpleImageProcessor:
    """Minimal Qwen-style image processor: resize (nearest) so that both sides are multiples of
    patch*merge, normalise to mean 0.5 / std 0.5, duplicate the frame ``temporal_patch_size``
    times and emit flattened patches in merge-block order with ``image_grid_thw``."""

    def __init__(self, patch_size: int = 16, merge_size: int = 2, temporal_patch_size: int = 2,
                 min_side: int | None = None):
        self.patch_size, self.merge_size, self.temporal_patch_size = patch_size, merge_size, temporal_patch_size
        self.min_side = min_side or patch_size * merge_size

    def preprocess(self, images, return_tensors="np"):
        import numpy as np

        p, m, tp = self.patch_size, self.merge_size, self.temporal_patch_size
        unit = p * m
        pix, grids = [], []
        for im in images:
            a = np.asarray(im, dtype=np.float32)
            if a.ndim == 2:
                a = np.stack([a] * 3, -1)
            if a.max() > 1.5:
                a = a / 255.0
            H, W = a.shape[:2]
            h = max(unit, int(round(H / unit)) * unit)
            w = max(unit, int(round(W / unit)) * unit)
            ri = (np.arange(h) * H / h).astype(int).clip(0, H - 1)
            ci = (np.arange(w) * W / w).astype(int).clip(0, W - 1)
            a = (a[ri][:, ci, :3] - 0.5) / 0.5
            a = np.transpose(a, (2, 0, 1))[None].repeat(tp, 0)            # [tp, C, h, w]
            gh, gw = h // p, w // p
            a = a.reshape(1, tp, 3, gh // m, m, p, gw // m, m, p)
            a = a.transpose(0, 3, 6, 4, 7, 2, 1, 5, 8)                     # [t, gh/m, gw/m, m, m, C, tp, p, p]
            pix.append(a.reshape(gh * gw, 3 * tp * p * p))
            grids.append([1, gh, gw])
        return {"pixel_values": np.concatenate(pix, 0).astype(np.float32),
                "image_grid_thw": np.asarray(grids, dtype=np.int64)}
