"""Normalisation layers of Qwen3.5 (reference: omegalax/models/qwen3_5/norms.py)."""
from __future__ import annotations

import torch
from torch import nn

from ...ops import functional as Fn
from ...ops import reference as R


from ...utils.profiling import scoped


class RMSNorm(nn.Module):
    """(1 + weight) * x / rms(x), fp32 arithmetic, weight initialised to zero."""

    def __init__(self, dim: int, eps: float = 1e-6, device=None, dtype=None):
        super().__init__()
        self.weight = nn.Parameter(torch.zeros(dim, device=device, dtype=dtype))
        self.eps = eps

    def reset_parameters(self):
        if self.weight.device.type != "meta":
            with torch.no_grad():
                self.weight.zero_()

    @scoped("rms_norm")
    def forward(self, x):
        return Fn.rmsnorm(x, self.weight, self.eps, one_plus=True)


class RMSNormGated(nn.Module):
    """weight * norm(x) in the input dtype, times silu(gate) evaluated in fp32."""

    def __init__(self, dim: int, eps: float = 1e-6, device=None, dtype=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))
        self.eps = eps

    def reset_parameters(self):
        if self.weight.device.type != "meta":
            with torch.no_grad():
                self.weight.fill_(1.0)

    @scoped("rms_norm_gated")
    def forward(self, x, gate):
        return Fn.rmsnorm_gated(x, self.weight, gate, self.eps)


class LayerNorm(nn.Module):
    """LayerNorm with bias, fp32 statistics (vision tower)."""

    def __init__(self, dim: int, eps: float = 1e-6, device=None, dtype=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(dim, device=device, dtype=dtype))
        self.eps = eps

    def reset_parameters(self):
        if self.weight.device.type != "meta":
            with torch.no_grad():
                self.weight.fill_(1.0)
                self.bias.zero_()

    @scoped("layer_norm")
    def forward(self, x):
        return Fn.layernorm(x, self.weight, self.bias, self.eps)
