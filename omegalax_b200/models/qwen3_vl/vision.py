"""Qwen3-VL vision tower: shared ViT with DeepStack mergers (post-shuffle norm) that returns
(merged features, [deepstack features...]).  Reference: omegalax/models/qwen3_vl/vision.py."""
from __future__ import annotations

from ..vision_common import VisionTower, vision_cu_seqlens  # noqa: F401
from .config import Qwen3VLVisionConfig


class VisionModel(VisionTower):
    def __init__(self, cfg: Qwen3VLVisionConfig, device=None, dtype=None):
        super().__init__(depth=cfg.depth, hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
                         num_heads=cfg.num_heads, patch_size=cfg.patch_size,
                         temporal_patch_size=cfg.temporal_patch_size, spatial_merge_size=cfg.spatial_merge_size,
                         in_channels=cfg.in_channels, out_hidden_size=cfg.out_hidden_size,
                         num_position_embeddings=cfg.num_position_embeddings, hidden_act=cfg.hidden_act,
                         deepstack_visual_indexes=cfg.deepstack_visual_indexes, device=device, dtype=dtype)
        self.cfg = cfg

    def forward(self, pixel_values, grid_thw, cu_seqlens=None):
        out = super().forward(pixel_values, grid_thw, cu_seqlens)
        return out if isinstance(out, tuple) else (out, [])
