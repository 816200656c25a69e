"""The step function: run a batch of (request, its next tokens) from the cache and return the
logits at the wanted places.  Everything above it (scheduler, generation, trace replay)
calls this one function; everything below it (model, cache, kernels) is called from here.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheManager, OutOfPages, StateNeed
from ..config import load_config
from ..csrc import ops
from ..parts.model import Model
from ..weights import RandomSource, SafetensorsSource, WeightSource
from .batch import EntryArrays, StepBatch, StepBuffers, StepEntry, pack_step

STATUS_TEXT = {1: "a token id outside the vocabulary reached the embedding kernel",
               2: "a block-table update pointed outside the table",
               3: "the cache write met a page number outside the pool",
               4: "attention met a page number outside the pool",
               5: "a wait on a copy barrier in the decode attention kernel ran out",
               6: "a wait on a barrier in the tcgen05 prompt attention kernel ran out",
               8: "a wait on a copy barrier in the weight-streaming product ran out",
               9: "a wait on a barrier in the paired tcgen05 product ran out"}


class ModelRunner:
    """A model on one GPU with its cache manager and the step function.

    The reference's engine owns the same things (src/engine/paged_generate_engine.cpp:17-97)
    but has three entry points — prefill, decode_one_step, decode_batch (:99-341) — where this
    has `step`.
    """

    # Graphs of "any step of T tokens" are kept for steps short enough that launching their kernels one
    # by one costs as much as running them, and for a bounded number of different T.
    MIXED_GRAPH_MAX_TOKENS = 1024
    MIXED_GRAPH_MAX_COUNT = 16

    def __init__(self, model: Model, page_size: int = 16, max_total_tokens: int = 4096,
                 max_requests: int = 64, max_tokens_per_step: int = 8192,
                 max_request_tokens: Optional[int] = None, use_graphs: bool = True):
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device: the engine has no CPU path")
        ops.configure_library_products()
        self.model = model
        self.plan = model.plan
        self.device = model.device
        limit = min(max_request_tokens or self.plan.max_position, self.plan.max_position)
        def make_cache():
            return CacheManager(
                model.stage_needs(), page_size, max_total_tokens, max_requests, max_request_tokens=limit,
                dtype=model.dtype, device=self.device,
                extra_state={"sampler": StateNeed((4,), "int32")})
        try:
            self.cache = make_cache()
        except torch.cuda.OutOfMemoryError:
            # The second, tiled copies of the decode weights are a convenience: the cache goes first.
            if ops.release_streaming() == 0:
                raise
            torch.cuda.empty_cache()
            self.cache = make_cache()
        self.buffers = StepBuffers(max_tokens_per_step, max_requests, len(self.cache.groups), self.device,
                                   preludes=model.step_preludes())
        # Tokens sampled by the step before, for entries whose last token the host has not read yet
        # (`StepEntry.feedback`); whoever samples writes them here.
        self.sampled = torch.zeros(max_requests, dtype=torch.int32, device=self.device)
        self.steps_run = 0
        # CUDA graphs for steps made only of single decoded tokens: one graph per batch size,
        # captured the second time that size is seen.  Only for models whose parts all say
        # they launch nothing but kernels on the current stream (no host reads, no host loops).
        self.use_graphs = use_graphs and all(
            getattr(b.mixer, "graph_safe", False) and getattr(b.feed_forward, "graph_safe", False)
            for b in model.blocks)
        self._graphs = {}
        self._mixed_graphs = True               # graphs for steps that are not all single decoded tokens
        # Parts that say `any_division_safe` read the step's per-entry arrays only through kernels that
        # take their work from a prelude's padded lists: one graph then serves every step of T tokens.
        # Parts that are only `graph_safe` may shape tensors by the number of entries, so their graphs
        # are kept per (tokens, entries).
        self._entries_free = all(
            getattr(b.mixer, "any_division_safe", False) and getattr(b.feed_forward, "any_division_safe", False)
            for b in model.blocks)
        self._mixed_count = 0
        self._graph_seen = {}
        self._graph_pool = None
        self._graph_weights = ops.streaming_generation()
        self.graph_replays = 0

    # ---- construction ----------------------------------------------------------------------
    @classmethod
    def from_folder(cls, model_dir: str, dtype="bfloat16", device="cuda", **kw) -> "ModelRunner":
        config = load_config(model_dir)
        model = Model(config.plan(), dtype=dtype, device=device)
        model.load_weights(SafetensorsSource(model_dir), where=model_dir)
        r = cls(model, **kw)
        r.config = config
        return r

    @classmethod
    def from_config(cls, config, seed: int = 0, dtype="bfloat16", device="cuda",
                    source: Optional[WeightSource] = None, **kw) -> "ModelRunner":
        """Random weights drawn on the device (for benchmarks); `source` overrides them."""
        model = Model(config.plan(), dtype=dtype, device=device)
        if source is None:
            store = torch.bfloat16 if model.dtype == torch.bfloat16 else torch.float32
            source = RandomSource(model.parameters(), seed, store, device=device)
        model.load_weights(source)
        r = cls(model, **kw)
        r.config = config
        return r

    # ---- requests --------------------------------------------------------------------------
    def admit(self) -> int:
        return self.cache.admit()

    def release(self, slot: int) -> None:
        self.cache.release(slot)

    # ---- the step --------------------------------------------------------------------------
    def prepare(self, entries: Sequence[StepEntry], state_writes=()) -> StepBatch:
        """Host half of a step: checks, pages, metadata upload, block-table updates.
        `state_writes`: [(name of a per-request state tensor of int32, slot, values)]: the values
        become that slot's row before the step's first kernel runs; they travel in the step's own
        upload, so admitting a request costs no copy of its own."""
        entries = list(entries)
        if not entries:
            raise ValueError("a step needs at least one entry")
        a = EntryArrays.of(entries)
        V, B = self.plan.vocab_size, len(entries)
        if len(np.unique(a.slot)) != B:
            twice = next(s for i, s in enumerate(a.slot.tolist()) if s in a.slot[:i])
            raise ValueError(f"slot {twice} appears twice in one step")
        if int(a.q_len.min()) == 0:
            raise ValueError("an entry needs at least one token")
        if int(a.fed.max()) >= self.sampled.numel():
            raise ValueError(f"feedback index {int(a.fed.max())} is outside the {self.sampled.numel()} sampled tokens")
        known = a.tokens
        if int(a.fed.max()) >= 0:                                 # an entry's last token may still be on the device
            known = np.delete(known, (np.cumsum(a.q_len) - 1)[a.fed >= 0])
        if len(known) and (int(known.min()) < 0 or int(known.max()) >= V):
            bad = int(known[(known < 0) | (known >= V)][0])
            raise ValueError(f"token id {bad} is outside the vocabulary [0, {V})")
        a.past = self.cache.lengths(a.slot)
        new_len = a.past + a.q_len
        if int(new_len.max()) > self.plan.max_position:
            raise ValueError(f"position {int(new_len.max()) - 1} exceeds max_position_embeddings {self.plan.max_position}")
        for e, p in zip(entries, a.past.tolist()):
            e.past = p
        try:
            self.cache.ensure_all(a.slot, new_len)                # for all of them, or nothing is taken
        except OutOfPages as err:
            raise OutOfPages(f"the step's tokens do not fit the free pages ({err})") from None
        writes = []
        for name, slot, values in state_writes:
            t = self.cache.state[name]
            if t.dtype != torch.int32 or len(values) != t[0].numel():
                raise ValueError(f"state {name!r} wants {t[0].numel()} int32 values per request")
            base = slot * t[0].numel()
            writes.append((np.arange(base, base + len(values), dtype=np.int64), np.asarray(values, dtype=np.int64)))
        batch = pack_step(self.buffers, entries, self.cache.drain_updates(), feedback=self.sampled, state_writes=writes,
                          arrays=a)
        region = self.buffers.last                              # where pack_step put this step
        counts = region.dev_view("counts")
        for (name, _, _), (at, n) in zip(state_writes, batch.state_ranges):
            o = region.off["state_index"][0]
            v = region.off["state_value"][0]
            ops.scatter_int32(self.cache.state[name].view(-1), region.dev[o + at:o + at + n], region.dev[v + at:v + at + n],
                              None, n, self.buffers.status)
        for g, group in enumerate(self.cache.groups):
            n = int(region.host_view("counts")[8 + g])
            if n:
                ops.scatter_int32(group.table_dev, region.dev_view(f"upd_index{g}", n),
                                  region.dev_view(f"upd_value{g}", n), counts[8 + g:9 + g], n,
                                  self.buffers.status)
        return batch

    def finish(self, batch: StepBatch) -> None:
        self.cache.commit_all(batch.entry_slots, batch.entry_new_len)
        self.steps_run += 1

    def forward(self, batch: StepBatch) -> torch.Tensor:
        """The device half of a step.  Steps are replayed as captured CUDA graphs of the same kernels
        where one graph can serve them: a step of B single decoded tokens that wants all B logits
        (one graph per B), and any other step of T tokens that wants at most one row per entry slot
        (one graph per T: its attention kernels run over padded work lists, so it does not matter how
        the T tokens are divided among requests; per (T, entries) for models with a part that does
        not say `any_division_safe`).  A graph is captured the second time its key is
        seen; everything else launches the kernels one by one.  A graph's logits tensor is reused by
        the next replay of that graph: read it (sample, copy) before stepping again."""
        if self.use_graphs:
            B = batch.num_tokens
            if self._graph_weights != ops.streaming_generation():   # the tiled weight copies a graph points at are gone
                self._graphs.clear()
                self._mixed_count = 0
                self._graph_weights = ops.streaming_generation()
            # The last member of a key: what the parts' launches depend on beyond the token count (the
            # decode attention's key splits grow with the longest cached length, in steps).
            if batch.max_q_len == 1 and batch.num_want == B:
                # a graph holds the device addresses of one layout
                key = (B, "decode", batch.layout, B, self.model.graph_variant(batch, False))
            elif self._mixed_graphs and batch.num_want <= batch.want_cap and B <= self.MIXED_GRAPH_MAX_TOKENS:
                # "none": a prompt portion that wants nothing has no output head in its graph
                key = (B, "any" if batch.num_want else "none", batch.layout, 0 if self._entries_free else batch.num_entries,
                       self.model.graph_variant(batch, True))
                if key not in self._graphs and self._mixed_count >= self.MIXED_GRAPH_MAX_COUNT:
                    key = None
            else:
                key = None
            if key is not None:
                g = self._graphs.get(key)
                if g is None:
                    seen = self._graph_seen.get(key, 0)
                    self._graph_seen[key] = seen + 1
                    if seen >= 1:
                        g = self._capture(batch, key)
                if g is not None:
                    g[0].replay()
                    self.graph_replays += 1
                    ops.launch_count += g[2]          # the kernels the graph holds ran again
                    return g[1] if key[1] == "decode" else g[1][:batch.num_want]
        return self.model.forward(batch, self.cache)

    def _capture(self, batch: StepBatch, key):
        # Launch choices inside a graph may depend on the step's lengths only as far as the parts'
        # `graph_variant` says (it is part of the key), not on how the tokens are divided, nor on how
        # many rows are wanted.
        real = (batch.num_want, batch.want_rows, batch.any_division)
        if key[1] != "decode":
            batch.any_division = True
            if key[1] == "any":
                batch.num_want = batch.want_cap
                batch.want_rows = self.buffers.last.dev_view("want_rows", batch.want_cap)
        cur = torch.cuda.current_stream()
        side = torch.cuda.Stream()
        side.wait_stream(cur)
        # The warm-up below runs the step for real and the first replay runs it again.  Keys and values
        # land in the same places with the same values both times; a mixer's fixed-size state would be
        # advanced twice, so it is put back in between.
        states = {k: t.clone() for k, t in self.cache.state.items() if isinstance(k, int)}
        with torch.cuda.stream(side):           # warm every kernel and library handle outside capture
            self.model.forward(batch, self.cache)
            for k, t in states.items():
                self.cache.state[k].copy_(t)
        cur.wait_stream(side)
        torch.cuda.synchronize()
        batch.tables.clear()                    # what the warm-up computed once for its layers: the graph must compute its own
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        graph = torch.cuda.CUDAGraph()
        before = ops.launch_count
        with torch.cuda.graph(graph, pool=self._graph_pool):
            logits = self.model.forward(batch, self.cache)
        kernels = ops.launch_count - before     # counted while capturing, not run
        ops.launch_count = before
        batch.num_want, batch.want_rows, batch.any_division = real
        self._graphs[key] = (graph, logits, kernels)
        self._mixed_count += key[1] != "decode"
        return self._graphs[key]

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run the entries' tokens as one batch; returns float32 [wanted, vocab] in the order of
        the entries and of each entry's `want`."""
        batch = self.prepare(entries)
        logits = self.forward(batch)
        self.finish(batch)
        return logits

    def check_status(self) -> None:
        """Raise if a kernel recorded a refused index or a wait that gave up (reads the step's
        status word and the matrix products' own; synchronises).  Both words are cleared."""
        for word in (self.buffers.status, ops.stream_status(self.device)):
            code, where = word.tolist()
            if code:
                word.zero_()
                raise RuntimeError(f"device status {code}: {STATUS_TEXT.get(code, 'unknown')} (at index {where})")
