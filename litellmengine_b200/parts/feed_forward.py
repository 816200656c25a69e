"""Feed-forward parts."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.specs import FeedForwardSpec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .registry import register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU:
    """down(silu(gate(x)) * up(x)), no biases (src/model/qwen3.cpp:143-152,
    src/ops/silu_and_mul.cu:44-46).  Gate and up are one fused product [g | u]."""

    graph_safe = True          # forward only launches kernels on the current stream
    any_division_safe = True   # and nothing in it is shaped by the number of entries of the step

    def __init__(self, spec: FeedForwardSpec, hidden_size: int, compute_dtype: torch.dtype, device):
        if spec.intermediate_size <= 0:
            raise ValueError("intermediate_size must be positive")
        self.hidden, self.inter, self.dtype = hidden_size, spec.intermediate_size, compute_dtype
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamSpec]:
        return {"gate_proj.weight": ParamSpec((self.inter, self.hidden)),
                "up_proj.weight": ParamSpec((self.inter, self.hidden)),
                "down_proj.weight": ParamSpec((self.hidden, self.inter))}

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        g, u = t["gate_proj.weight"], t["up_proj.weight"]
        dt = torch.float32 if torch.float32 in (g.dtype, u.dtype) else g.dtype
        self.w_gate_up = torch.cat([g.to(dt), u.to(dt)], dim=0).contiguous()
        self.w_down = t["down_proj.weight"].contiguous()
        ops.prepare_streaming(self.w_gate_up)       # a tiled copy for decode steps (bfloat16 on a GPU only)
        ops.prepare_streaming(self.w_down)

    supports_partials = True   # forward(x, partials_ok=True) may return an ops.PartialSum
    supports_residual = True   # forward(x, residual=h) may add its result to h itself and return None

    def forward(self, x: torch.Tensor, partials_ok: bool = False, residual: Optional[torch.Tensor] = None):
        act = ops.linear_silu_mul(x, self.w_gate_up, self.dtype)
        if residual is not None and ops.linear_into(act, self.w_down, residual):
            return None                                                               # joined the residual in the product
        return ops.linear(act, self.w_down, out_dtype=torch.float32, partials_ok=partials_ok)
