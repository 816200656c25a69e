"""Position encodings.  A position part owns how queries and keys are encoded by position.

Two ways to be one:
  * `rotation(batch)` returns a `Rotation` (the tables of a half-split rotation) or None (nothing
    is done to q and k): the attention mixer's fused kernel then normalises, rotates and writes
    the cache in one pass.
  * no `rotation` method, but `apply(q, k, batch) -> (q, k)`: float32 [T, heads, head_dim]
    tensors (k is None for a mixer without keys of its own) after the per-head norms, returned
    encoded.  The mixer runs the norms, this method, and the cache write as separate kernels,
    so an encoding of any kind needs no change to the mixer or to its kernels.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..config.specs import PositionSpec
from .registry import register_position


@dataclass
class Rotation:
    """What the fused kernel rotates by: pairs (i, i + rotary_dim/2) of a head by the angle
    float(position) * inv_freq[i]; `angles` is the step's table of their sines and cosines
    (float32 [T, rotary_dim/2, 2]) or None, in which case the kernel computes them."""
    inv_freq: torch.Tensor
    rotary_dim: int
    angles: Optional[torch.Tensor] = None


@register_position("none")
class NoPosition:
    def __init__(self, spec: PositionSpec, head_dim: int, device):
        pass

    def rotation(self, batch) -> Optional[Rotation]:
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

    def rotation(self, batch) -> Rotation:
        return Rotation(self.inv_freq, self.rotary_dim, self.angles(batch))

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
