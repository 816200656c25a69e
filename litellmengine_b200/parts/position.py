"""Position encodings.  A position part holds the tables a mixer's kernels need; the
rotation itself happens inside the mixer's fused kernel."""
from __future__ import annotations

import torch

from ..config.specs import PositionSpec
from .registry import register_position


@register_position("none")
class NoPosition:
    def __init__(self, spec: PositionSpec, head_dim: int, device):
        self.inv_freq = None
        self.rotary_dim = 0


@register_position("rope")
class RotaryPosition:
    """Half-split rotation: inv_freq[i] = theta ** (-(2 i) / rotary_dim), computed once in
    float32 with theta held as float32, as the reference does per call
    (src/layers/rotary.cu:81-83).  The angle float(pos) * inv_freq[i] and its sine and cosine
    are computed in 32-bit inside the kernel (src/layers/rotary.cu:101-105)."""

    def __init__(self, spec: PositionSpec, head_dim: int, device):
        rd = spec.rotary_dim or head_dim
        if rd <= 0 or rd % 2 != 0 or rd > head_dim:
            raise ValueError(f"rotary_dim {rd} must be even and at most head_dim {head_dim}")
        if not spec.theta > 0:
            raise ValueError("rope theta must be positive")
        self.rotary_dim = rd
        i = torch.arange(rd // 2, dtype=torch.float32)
        expo = -(2.0 * i) / torch.tensor(float(rd), dtype=torch.float32)
        self.inv_freq = torch.pow(torch.tensor(spec.theta, dtype=torch.float32), expo).to(device).contiguous()
