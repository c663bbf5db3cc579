"""RMSNorm, fused with the residual add that precedes it.

``y = x * rsqrt(mean(x^2) + eps) * w``: normalise first, multiply by the weight second, no ``1 + w``
and no bias (src/iian/graph.cpp:105-114).  The sum of squares and the residual sum are float32.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Norm, register_norm


@register_norm("rms_norm")
class RMSNorm(Norm):
    """params: ``size``, ``eps``."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.weight: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.size,), init="ones_jitter")}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].to(torch.float32).contiguous()     # exact widening; the kernel multiplies in float32

    def kernel_libraries(self):
        return ("elementwise",)

    def foldable(self):
        return (self.weight, self.eps) if self.weight is not None else None

    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], ctx) -> torch.Tensor:
        out = ctx.buf("normed", residual.shape, self.dtype)
        ops.kernels().add_rms_norm(residual, delta, self.weight, self.eps, out)
        return out
