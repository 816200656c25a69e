"""Registries of the kinds of parts a layer can be assembled from.

A part is a class built from its spec and the model's hidden size; it declares the tensors
it wants (`parameters`), receives them (`load`), and runs (`forward`).  No part knows which
model it is in.  Adding a kind is one `register_*` call; nothing else in the package
changes.  The interfaces:

  norm           __init__(spec: NormSpec, size: int)
                 parameters() -> {local name: ParamSpec}
                 load(tensors: {local name: tensor})
                 forward(x, out_dtype, delta=None, rows=None, write_sum=False) -> tensor
                     norm of x (+ delta); with write_sum the sum is stored back into x;
                     rows picks the rows to normalise.
  position       __init__(spec: PositionSpec, head_dim: int, device)
                 either rotation(batch) -> Rotation | None (the tables of a half-split rotation,
                 applied inside the attention mixer's fused kernel; None: nothing is done)
                 or apply(q, k, batch) -> (q, k) on float32 [T, heads, head_dim] after the
                 per-head norms (any other encoding; k is None for a mixer without keys)
  mixer          __init__(spec: MixerSpec, hidden_size: int, compute_dtype, device)
                 parameters(), load(tensors)
                 cache_need() -> PagedNeed | StateNeed | None
                 forward(x [T, hidden] compute dtype, ctx: StageContext) -> [T, hidden]
                 optional step_prelude() -> StepPrelude: work lists it wants built from a step's
                 entries once, in the step's own upload (found in ctx.batch.preludes[name])
  feed_forward   __init__(spec: FeedForwardSpec, hidden_size: int, compute_dtype, device)
                 parameters(), load(tensors)
                 forward(x [T, hidden]) -> [T, hidden]
  arrangement    a function (block, h, delta, ctx) -> (h, delta) wiring a layer's parts

In decode steps a product may be returned as `ops.PartialSum` (its k-splits, not yet added) to
a consumer that says it adds them itself: a norm with `accepts_partials = True` (its `delta`
may then be one), a feed-forward with `supports_partials = True` (it is then called with
`partials_ok=True`), a mixer through `ctx.partials_ok`.  Parts that say nothing never see one.

A mixer or feed-forward whose forward only launches kernels on the current stream (no host
reads, no loops over host data) may set the class attribute `graph_safe = True`; steps of a
model whose parts all do are replayed as CUDA graphs, one per (tokens, entries) of a step.  A
part in which nothing is shaped by the number of entries either (it reads the per-entry arrays
only inside kernels, and takes its work lists from a prelude that pads them) may also set
`any_division_safe = True`: one graph then serves every step of as many tokens.
"""
from __future__ import annotations

from typing import Callable, Dict

_KINDS: Dict[str, Dict[str, object]] = {"norm": {}, "position": {}, "mixer": {}, "feed_forward": {},
                                        "arrangement": {}}


def _register(family: str, kind: str):
    def deco(obj):
        _KINDS[family][kind] = obj
        return obj
    return deco


def register_norm(kind: str):
    return _register("norm", kind)


def register_position(kind: str):
    return _register("position", kind)


def register_mixer(kind: str):
    return _register("mixer", kind)


def register_feed_forward(kind: str):
    return _register("feed_forward", kind)


def register_arrangement(kind: str):
    return _register("arrangement", kind)


def unregister(family: str, kind: str) -> None:
    _KINDS[family].pop(kind, None)


def lookup(family: str, kind: str):
    try:
        return _KINDS[family][kind]
    except KeyError:
        raise KeyError(f"no {family} of kind {kind!r}; registered: {sorted(_KINDS[family])}") from None
