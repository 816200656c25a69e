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

    def angles(self, batch):
        return None


@register_position("rope")
class RotaryPosition:
    """Half-split rotation: inv_freq[i] = powf(theta, -(2 i) / rotary_dim) with theta and the
    exponent held as float32, as the reference computes per call (src/layers/rotary.cu:81-83).
    The table is made once, as the correctly rounded float32 power (the power taken in double
    precision of the float32 operands, then rounded): an inv_freq that is one unit in the last
    place off turns into an angle error of position * 6e-8, which is what separates one powf
    from another at long contexts.  The angle float(pos) * inv_freq[i] and its sine and cosine
    are computed in 32-bit inside the kernel (src/layers/rotary.cu:101-105)."""

    def __init__(self, spec: PositionSpec, head_dim: int, device):
        rd = spec.rotary_dim or head_dim
        if rd <= 0 or rd % 2 != 0 or rd > head_dim:
            raise ValueError(f"rotary_dim {rd} must be even and at most head_dim {head_dim}")
        if not spec.theta > 0:
            raise ValueError("rope theta must be positive")
        self.rotary_dim = rd
        i = torch.arange(rd // 2, dtype=torch.float32)
        expo = -(2.0 * i) / torch.tensor(float(rd), dtype=torch.float32)            # float32 quotient
        theta32 = torch.tensor(spec.theta, dtype=torch.float32)
        inv = torch.pow(theta32.double(), expo.double()).to(torch.float32)
        self.inv_freq = inv.to(device).contiguous()
        self._key = ("rope", float(spec.theta), rd)
        self._table_ok = rd == head_dim and head_dim in (64, 128)      # what the kernel that reads the table takes

    def angles(self, batch):
        """The step's table of sines and cosines, made by the first layer that asks and shared by
        all layers with the same theta and rotary_dim; None for steps of few tokens, whose kernels
        compute their own before they wait for the projection."""
        from ..csrc import ops
        tables = getattr(batch, "tables", None)
        if (tables is None or not self._table_ok or batch.num_tokens < ops.ROPE_TABLE_MIN_TOKENS
                or not self.inv_freq.is_cuda):
            return None
        if self._key not in tables:
            tables[self._key] = ops.rope_angles(batch.positions, self.inv_freq)
        return tables[self._key]
