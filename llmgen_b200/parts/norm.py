"""RMSNorm fused with the residual add that precedes it."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import Part
from .registry import register_norm
from .spec import INIT_ONE_PLUS_NORMAL, VECTOR, RMSNormSpec, WeightDecl


class RMSNorm(Part):
    """y = x / sqrt(mean(x^2) + eps) * (w + offset), all in float32, rounded once on store.

    Reference: src/backend/cpu/norm.zig:60-93 (which rounds x * r to bfloat16 before the
    gain; the single rounding here is closer to the float32 result)."""

    @staticmethod
    def weight_decls(spec: RMSNormSpec):
        return [WeightDecl(spec.weight, (spec.dim,), VECTOR, INIT_ONE_PLUS_NORMAL)]

    @staticmethod
    def kernel_modules(spec):
        return ("elementwise",)

    def __init__(self, spec: RMSNormSpec, weights, dtype, device):
        self.spec = spec
        self.weight = weights.device_tensor(spec.weight, dtype, device)   # float32 [dim]
        self.eps = float(spec.eps)
        self.offset = float(spec.weight_offset)

    def add_norm(self, resid: torch.Tensor, delta: Optional[torch.Tensor], out: torch.Tensor,
                 rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        ops.add_rmsnorm(resid, delta, self.weight, out, self.eps, self.offset, rows=rows)
        return out


register_norm("rmsnorm", RMSNorm)
