"""A layer put together from its parts, and the arrangements that wire them."""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..config.specs import BlockSpec
from ..weights.loader import ParamSpec
from .context import StageContext
from .registry import lookup, register_arrangement


class Block:
    """Holds one layer's mixer, feed-forward and norms, each chosen by the layer's spec."""

    def __init__(self, spec: BlockSpec, hidden_size: int, compute_dtype: torch.dtype, device):
        self.spec = spec
        self.dtype = compute_dtype
        self.mixer_norm = lookup("norm", spec.mixer_norm.kind)(spec.mixer_norm, hidden_size)
        self.feed_forward_norm = lookup("norm", spec.feed_forward_norm.kind)(spec.feed_forward_norm, hidden_size)
        self.mixer = lookup("mixer", spec.mixer.kind)(spec.mixer, hidden_size, compute_dtype, device)
        self.feed_forward = lookup("feed_forward", spec.feed_forward.kind)(
            spec.feed_forward, hidden_size, compute_dtype, device)
        self.arrangement = lookup("arrangement", spec.arrangement)

    def _children(self):
        s = self.spec
        return ((s.mixer_norm_name, self.mixer_norm), (s.mixer.weight_prefix, self.mixer),
                (s.feed_forward_norm_name, self.feed_forward_norm),
                (s.feed_forward.weight_prefix, self.feed_forward))

    def parameters(self) -> Dict[str, ParamSpec]:
        out = {}
        for prefix, part in self._children():
            for name, p in part.parameters().items():
                out[f"{prefix}.{name}"] = p
        return out

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        for prefix, part in self._children():
            part.load({n[len(prefix) + 1:]: t for n, t in tensors.items() if n.startswith(prefix + ".")})

    def forward(self, h: torch.Tensor, delta: Optional[torch.Tensor], ctx: StageContext
                ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        return self.arrangement(self, h, delta, ctx)


@register_arrangement("pre_norm")
def pre_norm(block: Block, h: torch.Tensor, delta: Optional[torch.Tensor], ctx: StageContext):
    """h += mixer(norm1(h)); h += ffn(norm2(h))  (src/model/qwen3.cpp:948-968).

    `h` is the float32 residual stream; `delta` is the previous layer's feed-forward output
    that has not been added yet (None if nothing is pending).  Each add is fused into the norm
    that follows it, so the layer returns its own feed-forward output as the next pending delta,
    unless the part added it to `h` itself (in the epilogue of its last product).
    """
    from ..csrc import ops
    if not getattr(block.mixer_norm, "accepts_partials", False):
        delta = ops.as_tensor(delta)
    x = block.mixer_norm.forward(h, block.dtype, delta=delta, write_sum=delta is not None)
    ctx.partials_ok = getattr(block.feed_forward_norm, "accepts_partials", False)
    ctx.residual = h                                            # a part may add its result here itself and return None
    a = block.mixer.forward(x, ctx)
    y = block.feed_forward_norm.forward(h, block.dtype, delta=a, write_sum=a is not None)
    extra = {}
    if getattr(block.feed_forward, "supports_partials", False):
        extra["partials_ok"] = True                             # the next norm (or `pre_norm` above) adds the splits
    if getattr(block.feed_forward, "supports_residual", False):
        extra["residual"] = h
    f = block.feed_forward.forward(y, **extra)
    return h, f
