"""ChatML serialisation and encoding of Qwen chat examples (reference: omegalax/data/qwen3_encoding.py).

A message is rendered as ``<|im_start|>{role}\\n{content}<|im_end|>\\n``; an image block becomes
``<|vision_start|>`` + ``<|image_pad|>`` * (t * h/m * w/m) + ``<|vision_end|>``.  Because the
delimiters are special tokens, per-message token counts are exactly additive, which is what
the chunk index relies on.
"""
from __future__ import annotations

from typing import Any

import numpy as np


def build_chatml_text(messages, image_grids, merge_size: int) -> str:
    parts, k = [], 0
    for msg in messages:
        parts.append(f"<|im_start|>{msg['role']}\n")
        content = msg["content"]
        if isinstance(content, str):
            parts.append(content)
        else:
            for block in content:
                if block["type"] == "text":
                    parts.append(block["text"])
                elif block["type"] == "image":
                    t, h, w = image_grids[k]
                    k += 1
                    parts.append("<|vision_start|>" + "<|image_pad|>" * (t * (h // merge_size) * (w // merge_size))
                                 + "<|vision_end|>")
        parts.append("<|im_end|>\n")
    return "".join(parts)


def extract_images(messages) -> list:
    """Images of the structured-content blocks: PIL images, numpy arrays, paths or urls."""
    out = []
    for msg in messages:
        content = msg["content"]
        if isinstance(content, str):
            continue
        for block in content:
            if block.get("type") != "image":
                continue
            src = block.get("image", block.get("url"))
            if isinstance(src, (str, bytes)) or hasattr(src, "__fspath__"):
                from PIL import Image

                src = Image.open(src)
            out.append(src)
    return out


def _message_has_images(message) -> bool:
    c = message.get("content", "")
    return (not isinstance(c, str)) and any(b.get("type") == "image" for b in c)


def encode_qwen_messages(messages, *, tokenizer, image_processor=None, include_pixels: bool = False) -> dict:
    grids, out = [], {}
    if image_processor is not None:
        imgs = extract_images(messages)
        if imgs:
            proc = image_processor.preprocess(imgs, return_tensors="np")
            out["image_grid_thw"] = np.asarray(proc["image_grid_thw"])
            if include_pixels:
                out["pixel_values"] = np.asarray(proc["pixel_values"])
            grids = [tuple(int(v) for v in row) for row in out["image_grid_thw"].tolist()]
    merge = int(getattr(image_processor, "merge_size", 1))
    text = build_chatml_text(messages, grids, merge)
    out["input_ids"] = np.asarray(tokenizer.encode(text, add_special_tokens=False), dtype=np.int32)
    return out


def make_message_length_fn(tokenizer, image_processor=None):
    """``message -> {"length", "vision_tokens", "vision_patches", "num_images", "image_grid_thw"}``
    for ``build_chunk_index``."""
    merge = int(getattr(image_processor, "merge_size", 1)) if image_processor else 1

    def measure(message) -> dict[str, Any]:
        if image_processor is None and _message_has_images(message):
            raise ValueError("Encountered image content in message but no image_processor was provided. "
                             "Pass image_processor= to make_message_length_fn.")
        enc = encode_qwen_messages([message], tokenizer=tokenizer, image_processor=image_processor)
        grid = enc.get("image_grid_thw", np.empty((0, 3), dtype=np.int64))
        vt = sum(int(t) * (int(h) // merge) * (int(w) // merge) for t, h, w in grid)
        vp = sum(int(t) * int(h) * int(w) for t, h, w in grid)
        return {"length": int(len(enc["input_ids"])), "vision_tokens": vt, "vision_patches": vp,
                "num_images": int(grid.shape[0]), "image_grid_thw": np.asarray(grid).tolist()}

    return measure
