"""Qwen3.5 vision tower (reference: omegalax/models/qwen3_5/vision.py).  The patch embedding
is a 3-D convolution with kernel == stride, i.e. a linear map over flattened patches; the
loader flattens the HF Conv3d weight (O, C, T, H, W) to (O, C*T*H*W)."""
from __future__ import annotations

from ..vision_common import VisionTower, token_spatial_coords, vision_cu_seqlens  # noqa: F401
from .config import Qwen3_5VisionConfig


class VisionModel(VisionTower):
    def __init__(self, cfg: Qwen3_5VisionConfig, device=None, dtype=None):
        super().__init__(depth=cfg.depth, hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
                         num_heads=cfg.num_heads, patch_size=cfg.patch_size,
                         temporal_patch_size=cfg.temporal_patch_size, spatial_merge_size=cfg.spatial_merge_size,
                         in_channels=cfg.in_channels, out_hidden_size=cfg.out_hidden_size,
                         num_position_embeddings=cfg.num_position_embeddings, hidden_act="gelu_pytorch_tanh",
                         device=device, dtype=dtype)
        self.cfg = cfg
