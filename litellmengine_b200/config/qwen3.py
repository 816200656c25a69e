"""Typed configuration of the Qwen3 dense decoder, read from its config.json keys.

Keys, defaults and checks follow the reference: required keys and the
`Missing required config field: <key>` message are src/model/model_config.cpp:13-20,45-51;
optional keys and their defaults are src/model/model_config.cpp:53-87; the value
checks are src/model/qwen3.cpp:19-75.  Keys the reference never reads but whose
non-default value would change the arithmetic (`hidden_act`, `attention_bias`,
`rope_scaling`, `use_sliding_window`) are read here and refused when they ask
for something that is not built, instead of being silently ignored.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Any, Dict

from .registry import ConfigError, register_architecture
from .specs import (BlockSpec, FeedForwardSpec, MixerSpec, ModelPlan, NormSpec, PositionSpec,
                    StageSpec)

_MISSING = object()


def _get(d: Dict[str, Any], key: str, kind, default=_MISSING):
    if key not in d or d[key] is None:
        if default is _MISSING:
            raise ConfigError(f"Missing required config field: {key}")
        return default
    v = d[key]
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v == int(v):
                return int(v)
            raise ConfigError(f"config field {key} must be an integer, got {v!r}")
        return v
    if kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config field {key} must be a number, got {v!r}")
        return float(v)
    if kind is bool:
        if not isinstance(v, bool):
            raise ConfigError(f"config field {key} must be true or false, got {v!r}")
        return v
    if kind is str:
        if not isinstance(v, str):
            raise ConfigError(f"config field {key} must be a string, got {v!r}")
        return v
    raise TypeError(kind)


@register_architecture("Qwen3ForCausalLM")
@dataclass(frozen=True)
class Qwen3Config:
    model_type: str
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int = 32768
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = False
    torch_dtype: str = "bfloat16"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Qwen3Config":
        model_type = _get(d, "model_type", str)
        vocab = _get(d, "vocab_size", int)
        hidden = _get(d, "hidden_size", int)
        inter = _get(d, "intermediate_size", int)
        layers = _get(d, "num_hidden_layers", int)
        heads = _get(d, "num_attention_heads", int)
        if heads <= 0:
            raise ConfigError("Qwen3 config num_attention_heads must be positive")
        kv_heads = _get(d, "num_key_value_heads", int, heads)
        head_dim = _get(d, "head_dim", int, hidden // heads)
        cfg = cls(
            model_type=model_type, vocab_size=vocab, hidden_size=hidden,
            intermediate_size=inter, num_hidden_layers=layers,
            num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
            max_position_embeddings=_get(d, "max_position_embeddings", int, 32768),
            rms_norm_eps=_get(d, "rms_norm_eps", float, 1e-6),
            rope_theta=_get(d, "rope_theta", float, 10000.0),
            tie_word_embeddings=_get(d, "tie_word_embeddings", bool, False),
            torch_dtype=_get(d, "torch_dtype", str, _get(d, "dtype", str, "bfloat16")),
        )
        act = _get(d, "hidden_act", str, "silu")
        if act != "silu":
            raise ConfigError(f"Qwen3 config hidden_act={act!r} is not built (only 'silu')")
        if _get(d, "attention_bias", bool, False):
            raise ConfigError("Qwen3 config attention_bias=true is not built")
        if d.get("rope_scaling") is not None:
            raise ConfigError("Qwen3 config rope_scaling is not built (must be null or absent)")
        if _get(d, "use_sliding_window", bool, False):
            raise ConfigError("Qwen3 config use_sliding_window=true is not built")
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                    "num_attention_heads", "num_key_value_heads", "head_dim",
                    "max_position_embeddings"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"Qwen3 config {key} must be positive")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                "Qwen3 config num_attention_heads must be divisible by num_key_value_heads")
        if self.head_dim % 2 != 0:
            raise ConfigError("Qwen3 config head_dim must be even (rotation works on pairs)")
        if not self.rms_norm_eps > 0.0:
            raise ConfigError("Qwen3 config rms_norm_eps must be positive")
        if not self.rope_theta > 0.0:
            raise ConfigError("Qwen3 config rope_theta must be positive")

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        d["architectures"] = [self.architecture]
        d["hidden_act"] = "silu"
        d["attention_bias"] = False
        d["rope_scaling"] = None
        d["use_sliding_window"] = False
        return d

    def plan(self) -> ModelPlan:
        """Every layer is the same pre-norm block (src/model/qwen3.cpp:879-968):
        RMSNorm, grouped-query attention with per-head q/k RMSNorm and half-split
        rotation (src/model/qwen3.cpp:357-449), RMSNorm, SwiGLU
        (src/model/qwen3.cpp:143-152); then a final RMSNorm and the output head
        (src/model/qwen3.cpp:1278,1501)."""
        norm = NormSpec(kind="rmsnorm", eps=self.rms_norm_eps)
        blocks = []
        for i in range(self.num_hidden_layers):
            mixer = MixerSpec(
                kind="attention",
                num_heads=self.num_attention_heads,
                num_kv_heads=self.num_key_value_heads,
                head_dim=self.head_dim,
                qk_norm=norm,
                position=PositionSpec(kind="rope", theta=self.rope_theta, rotary_dim=self.head_dim),
                window=None,
            )
            ffn = FeedForwardSpec(kind="swiglu", intermediate_size=self.intermediate_size)
            blocks.append(BlockSpec(
                arrangement="pre_norm", mixer=mixer, feed_forward=ffn,
                mixer_norm=norm, feed_forward_norm=norm,
                weight_prefix=f"model.layers.{i}",
            ))
        plan = ModelPlan(
            hidden_size=self.hidden_size, vocab_size=self.vocab_size,
            blocks=tuple(blocks), order=tuple(StageSpec(block=i) for i in range(self.num_hidden_layers)),
            final_norm=norm, tie_word_embeddings=self.tie_word_embeddings,
            max_position=self.max_position_embeddings,
        )
        plan.validate()
        return plan
