"""Normalisation parts."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.specs import NormSpec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .registry import register_norm


@register_norm("rmsnorm")
class RMSNorm:
    """out = v * rsqrt(mean(v^2) + eps) * weight with v = x (+ delta), everything in 32-bit
    (src/layers/rms_norm.cu:77-93).  The weight multiplies directly (no 1 + w)."""

    accepts_partials = True    # `delta` may be an ops.PartialSum: the kernel adds the k-splits as it reads

    def __init__(self, spec: NormSpec, size: int):
        self.eps = float(spec.eps)
        self.size = size
        self.weight: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.size,), role="scale", init=("one_plus_normal", 0.01))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].contiguous()

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype, delta: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None, write_sum: bool = False) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps, out_dtype, delta=delta, rows=rows, write_sum=write_sum)
