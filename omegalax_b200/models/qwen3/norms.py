"""RMSNorm module (fp32 statistics, scale applied in fp32; reference: qwen3/norms.py)."""
from __future__ import annotations

import torch
from torch import nn

from ...ops import functional as Fn


from ...utils.profiling import scoped


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, *, one_plus: bool = False,
                 scale_in_dtype: bool = False, device=None, dtype=None):
        super().__init__()
        init = torch.zeros if one_plus else torch.ones
        self.weight = nn.Parameter(init(dim, device=device, dtype=dtype))
        self.eps, self.one_plus, self.scale_in_dtype = eps, one_plus, scale_in_dtype

    def reset_parameters(self):
        if self.weight.device.type != "meta":
            with torch.no_grad():
                self.weight.fill_(0.0 if self.one_plus else 1.0)

    @scoped("rms_norm")
    def forward(self, x):
        return Fn.rmsnorm(x, self.weight, self.eps, self.one_plus, self.scale_in_dtype)
