"""A model built from a `ModelPlan`: embedding, stages, final norm, output head."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.specs import ModelPlan
from ..csrc import ops
from ..weights.loader import ParamSpec, WeightSource, check_source, fetch_tensor
from .block import Block
from .context import StageContext
from .registry import lookup


def _compute_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        dt = name
    else:
        dt = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
              "fp32": torch.float32}.get(str(name))
    if dt not in (torch.bfloat16, torch.float32):
        raise ValueError(f"dtype {name!r}: choose bfloat16 or float32")
    return dt


class Model:
    """Runs a step's tokens through the stages and returns logits at the wanted rows.

    The residual stream is float32 in both run modes; matrix products, activations between
    kernels and the cache are in the compute dtype (bfloat16 or float32); logits are float32.
    """

    def __init__(self, plan: ModelPlan, dtype="bfloat16", device="cuda"):
        plan.validate()
        self.plan = plan
        self.dtype = _compute_dtype(dtype)
        self.device = torch.device(device)
        self.blocks: List[Block] = [Block(b, plan.hidden_size, self.dtype, self.device) for b in plan.blocks]
        self.final_norm = lookup("norm", plan.final_norm.kind)(plan.final_norm, plan.hidden_size)
        self.embedding: Optional[torch.Tensor] = None
        self.output: Optional[torch.Tensor] = None

    # ---- weights -------------------------------------------------------------------------
    def parameters(self) -> Dict[str, ParamSpec]:
        p = self.plan
        out = {p.embedding_name: ParamSpec((p.vocab_size, p.hidden_size))}
        for spec, block in zip(p.blocks, self.blocks):
            for name, ps in block.parameters().items():
                out[f"{spec.weight_prefix}.{name}"] = ps
        out[p.final_norm_name] = self.final_norm.parameters()["weight"]
        out[p.output_name] = ParamSpec((p.vocab_size, p.hidden_size),
                                       optional_alias=p.embedding_name if p.tie_word_embeddings else None)
        return out

    def load_weights(self, source: WeightSource, where: str = "") -> None:
        """Check the whole source first (one error for everything wrong), then bind part by
        part so that at most one layer's unfused tensors are alive at a time."""
        p = self.plan
        params = self.parameters()
        aliased = check_source(params, source, where)
        if self.dtype == torch.bfloat16:               # one decision for all of the model's matrices
            ops.begin_model(sum(2 * ps.shape[0] * ps.shape[1] for n, ps in params.items()
                                if len(ps.shape) == 2 and n not in aliased), self.device)
        get = lambda n: fetch_tensor(source, n, params[n], self.dtype, self.device)
        self.embedding = get(p.embedding_name).contiguous()
        for spec, block in zip(p.blocks, self.blocks):
            block.load({n: get(f"{spec.weight_prefix}.{n}") for n in block.parameters()})
        self.final_norm.load({"weight": get(p.final_norm_name)})
        self.output = self.embedding if p.output_name in aliased else get(p.output_name).contiguous()
        ops.prepare_streaming(self.output)          # a tiled copy of the output head for decode steps

    def stage_needs(self) -> list:
        needs = []
        for st in self.plan.order:
            if st.cache_from is not None:
                needs.append(("borrow", st.cache_from))
            else:
                needs.append(self.blocks[st.block].mixer.cache_need())
        return needs

    def step_preludes(self) -> list:
        """The `StepPrelude`s the parts of this model offer (a part offers one through an optional
        `step_prelude()` method)."""
        out = []
        for b in self.blocks:
            for part in (b.mixer, b.feed_forward):
                make = getattr(part, "step_prelude", None)
                if make is not None:
                    out.append(make())
        return out

    def graph_variant(self, batch, padded: bool) -> tuple:
        """What the parts' kernel choices for this step depend on beyond the number of tokens: a part
        whose launches vary with the step's lengths says so through an optional
        `graph_variant(batch, padded)` (any hashable; `padded`: the step would be captured over its
        preludes' padded lists).  Steps with equal variants can replay one captured graph.  Parts that
        give the same `graph_variant_group` choose alike and are asked once."""
        out, seen = [], set()
        for b in self.blocks:
            for part in (b.mixer, b.feed_forward):
                ask = getattr(part, "graph_variant", None)
                group = getattr(part, "graph_variant_group", None)
                if ask is None or (group is not None and group in seen):
                    continue
                seen.add(group)
                out.append(ask(batch, padded))
        return tuple(out)

    def weight_bytes(self) -> int:
        """Bytes of every weight tensor one decode step reads (a tied head counts twice: the
        embedding rows read are negligible, the head is read whole)."""
        seen, total = set(), 0

        def add(t):
            nonlocal total
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        for b in self.blocks:
            for part in (b.mixer, b.feed_forward):
                for v in vars(part).values():
                    if isinstance(v, torch.Tensor) and v.dim() == 2:
                        add(v)
        add(self.output)
        return total

    # ---- forward ---------------------------------------------------------------------------
    def forward(self, batch, cache) -> torch.Tensor:
        """batch: StepBatch already on the device; cache: CacheManager.  Returns float32
        [batch.num_want, vocab] (an empty tensor when nothing is wanted)."""
        with ops.bound_stream():                       # one stream for the whole pass, looked up once
            h = ops.embedding(batch.token_ids, self.embedding, batch.status, feedback=getattr(batch, "feedback", None))
            delta = None
            for s, st in enumerate(self.plan.order):
                block = self.blocks[st.block]
                h, delta = block.forward(h, delta, self.stage_context(s, batch, cache))
            if batch.num_want == 0:
                return torch.empty((0, self.plan.vocab_size), dtype=torch.float32, device=self.device)
            if not getattr(self.final_norm, "accepts_partials", False):
                delta = ops.as_tensor(delta)
            hn = self.final_norm.forward(h, self.dtype, delta=delta, rows=batch.want_rows)
            return ops.linear(hn, self.output, out_dtype=torch.float32)

    def stage_context(self, s: int, batch, cache) -> StageContext:
        st = self.plan.order[s]
        kv = table = keys = values = None
        if s in cache.stage_group:
            kv, table, _ = cache.stage_cache(s)
            keys, values = cache.stage_pages(s)
        return StageContext(batch=batch, stage=s, cache=kv, block_table=table, page_size=cache.page_size,
                            writes_cache=st.cache_from is None, state=cache.state.get(s), status=batch.status,
                            cache_keys=keys, cache_values=values)


def model_parameters(plan: ModelPlan) -> Dict[str, ParamSpec]:
    """The tensors a model of this plan wants, without building anything on a device."""
    return Model(plan, dtype="float32", device="meta").parameters()


def build_model(config, dtype="bfloat16", device="cuda") -> Model:
    return Model(config.plan(), dtype=dtype, device=device)
