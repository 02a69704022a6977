"""RMSNorm as a part: y = round(x * rsqrt(mean(x^2) + eps)) * w, statistics in 32-bit.

Formula and rounding points of the reference: src/ops/rms_norm.cu:87-120 (eps inside
the root, the weight multiplies directly).  The optional `delta` fuses the residual
sum of src/ops/elementwise.cu:30-34 into the same pass.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import Part, register_part


class RMSNorm(Part):
    def __init__(self, size: int, eps: float):
        self.size, self.eps = int(size), float(eps)
        self.weight = None

    def weight_specs(self, name: str) -> dict:
        return {name: WeightSpec((self.size,), "norm")}

    def bind(self, weights: dict, name: str, dtype, device) -> None:
        # a scale vector is used in 32-bit whatever it was stored in (exact for bfloat16)
        self.weight = weights[name].to(device=device, dtype=torch.float32).contiguous()

    def __call__(self, x: torch.Tensor, out: torch.Tensor, delta=None) -> torch.Tensor:
        return ops.rms_norm(x, self.weight, self.eps, out, delta)


register_part("norm", "rms_norm", RMSNorm)
