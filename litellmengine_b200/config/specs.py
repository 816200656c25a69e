"""Typed descriptions of the parts a model is assembled from.

A model is data: a list of distinct layers (`BlockSpec`), each naming its
mixer, feed-forward, norms and position encoding with every size and constant
as a field, and an `order` list saying which layer runs when.  Nothing here
knows about a particular architecture; an architecture's config class turns its
own config.json keys into a `ModelPlan` (see `config/qwen3.py`).

The reference hard-wires one arrangement (src/model/qwen3.cpp:841-1059) and one
set of sizes for all layers (src/model/qwen3.cpp:1067-1071); here the same
arrangement is one value of `BlockSpec.arrangement`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """A normalisation over the last dimension.  kind 'rmsnorm': x*rsqrt(mean(x^2)+eps)*w."""
    kind: str
    eps: float


@dataclass(frozen=True)
class PositionSpec:
    """How a mixer encodes token positions.

    kind 'rope': half-split rotation of pairs (i, i+rotary_dim/2) by the angle
    position * theta**(-2i/rotary_dim).  kind 'none': no encoding.
    `params` carries what other kinds need.
    """
    kind: str
    theta: float = 10000.0
    rotary_dim: int = 0
    params: Tuple[Tuple[str, Any], ...] = ()


@dataclass(frozen=True)
class MixerSpec:
    """The token-mixing part of a layer.

    kind 'attention': grouped-query causal attention over the paged cache.
    `window` = None attends to every earlier key; an integer w attends to the
    last w keys (the query's own included).  `has_kv` = False makes a mixer that
    projects only queries and reads the keys and values another stage wrote (the
    stage that runs it must then name that stage in `cache_from`).  `params`
    carries what other kinds of mixer need.
    """
    kind: str
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    qk_norm: Optional[NormSpec] = None
    position: PositionSpec = PositionSpec(kind="none")
    window: Optional[int] = None
    scale: Optional[float] = None          # None = 1/sqrt(head_dim)
    has_kv: bool = True
    weight_prefix: str = "self_attn"
    params: Tuple[Tuple[str, Any], ...] = ()


@dataclass(frozen=True)
class FeedForwardSpec:
    """The per-token part of a layer.  kind 'swiglu': down(silu(gate(x)) * up(x))."""
    kind: str
    intermediate_size: int = 0
    weight_prefix: str = "mlp"
    params: Tuple[Tuple[str, Any], ...] = ()


@dataclass(frozen=True)
class BlockSpec:
    """One layer: which parts it has and how they are wired.

    arrangement 'pre_norm': h += mixer(norm1(h)); h += ffn(norm2(h)).
    """
    arrangement: str
    mixer: MixerSpec
    feed_forward: FeedForwardSpec
    mixer_norm: NormSpec
    feed_forward_norm: NormSpec
    weight_prefix: str = ""
    mixer_norm_name: str = "input_layernorm"
    feed_forward_norm_name: str = "post_attention_layernorm"


@dataclass(frozen=True)
class StageSpec:
    """One entry of the run order: which layer runs, and whose cache it uses.

    A layer named by two stages shares its weights between them, but each stage
    has a cache (or state) of its own, unless `cache_from` names an EARLIER stage
    (by its index in the order) whose cache this stage reads without writing.
    """
    block: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelPlan:
    """Everything needed to build a model: sizes, layers, their order, names."""
    hidden_size: int
    vocab_size: int
    blocks: Tuple[BlockSpec, ...]
    order: Tuple[StageSpec, ...]            # the layers in the order they run; may repeat
    final_norm: NormSpec
    tie_word_embeddings: bool
    max_position: int
    embedding_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm.weight"
    output_name: str = "lm_head.weight"

    def validate(self) -> None:
        if self.hidden_size <= 0 or self.vocab_size <= 0:
            raise ValueError("hidden_size and vocab_size must be positive")
        if not self.blocks:
            raise ValueError("a model needs at least one layer")
        if not self.order:
            raise ValueError("the run order is empty")
        for s, st in enumerate(self.order):
            if not 0 <= st.block < len(self.blocks):
                raise ValueError(f"stage {s} names layer {st.block}, but there are {len(self.blocks)} layers")
            mixer = self.blocks[st.block].mixer
            if st.cache_from is not None:
                if not 0 <= st.cache_from < s:
                    raise ValueError(f"stage {s}: cache_from={st.cache_from} is not an earlier stage")
                if self.order[st.cache_from].cache_from is not None:
                    raise ValueError(f"stage {s}: cache_from={st.cache_from} itself borrows a cache")
            elif not mixer.has_kv:
                raise ValueError(f"stage {s}: its mixer writes no keys and values, so cache_from must be set")
