"""RMSNorm, fused with the residual addition that precedes it.

y = (x * rsqrt(mean(x^2) + eps)) * w, statistics in float
(src/kernels/layernorm.cu:20-23,41,48).  ``eps`` is a parameter; the reference
passes the literal 1e-6 at every call (src/model/qwen.cpp:303,312,322).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import Norm, ParamSpec, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, size: int, eps: float, dtype, device):
        if size <= 0 or not eps > 0:
            raise ValueError(f"rmsnorm: size {size} and eps {eps} must be positive")
        self.size, self.eps = size, float(eps)
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.size,), "gain")}

    def load_params(self, tensors):
        self.weight = tensors["weight"]

    def split(self):
        return (self.weight, self.eps) if self.weight is not None and self.weight.dtype == torch.float32 else None

    def forward(self, residual, delta, out, row_index=None):
        ops.add_rmsnorm(residual, delta, self.weight, out, self.eps, row_index)
