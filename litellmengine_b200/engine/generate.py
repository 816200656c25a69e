"""The Python entry point: `PagedGenerateEngine`, named and shaped after the reference's
class of that name (include/engine/paged_generate_engine.hpp:14-87): `add_request`,
`generate_until_finished`, `finished`, `request`, `release_request`.  Where the reference
has `prefill`, `decode_one_step` and `decode_batch`, this has one `step()` that runs
whatever the scheduler picked — prompt portions and decode tokens in the same batch — and
`run()` that steps until every request is finished.

Steps are pipelined by default: `step()` launches the next batch before it reads the tokens
of the one before, so the device never waits for the host's scheduling and packing.  A
request's next token then reaches the following step's embedding straight from the device
buffer it was sampled into (`StepEntry.feedback`); the host reads it one step late, which
is when finished requests are noticed.  `pipelined=False` reads every step's tokens before
the next is planned, as the reference does.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..sampling import Sampler
from ..sampling.sampler import slot_state_row
from .batch import StepEntry
from .request import GenerationRequest
from .runner import ModelRunner
from .scheduler import ScheduledPortion, Scheduler


class PagedGenerateEngine:
    def __init__(self, model, dtype: str = "bfloat16", device: str = "cuda:0", page_size: int = 16,
                 max_total_tokens: int = 8192, max_requests: int = 64, max_tokens_per_step: int = 8192,
                 chunk: Optional[int] = None, verbose: bool = False, seed: int = 0, pipelined: bool = True):
        """`model`: a model folder (config.json + *.safetensors), a typed configuration (random
        weights from `seed`, drawn on the device), or a ready `ModelRunner`."""
        if isinstance(model, ModelRunner):
            self.runner = model
        else:
            kw = dict(dtype=dtype, device=device, page_size=page_size, max_total_tokens=max_total_tokens,
                      max_requests=max_requests, max_tokens_per_step=max_tokens_per_step)
            if isinstance(model, str):
                self.runner = ModelRunner.from_folder(model, **kw)
            else:
                self.runner = ModelRunner.from_config(model, seed=seed, **kw)
        self.scheduler = Scheduler(self.runner.cache, self.runner.buffers.max_tokens, chunk)
        self.sampler = Sampler(self.runner.cache.state["sampler"])
        self.verbose = verbose
        self.pipelined = pipelined
        n = self.runner.buffers.max_entries
        self._tokens_pinned = [torch.empty(n, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._read_done = [torch.cuda.Event() for _ in range(2)]
        self._launched = 0
        self._in_flight = None            # (plan, requests that sample, which pinned buffer) of the launched step

    # ---- the reference's surface -------------------------------------------------------------
    def add_request(self, prompt_ids: Sequence[int], max_new_tokens: int, eos_token_id: int = -1,
                    temperature: float = 0.0, seed: int = 0) -> int:
        return self.scheduler.add(prompt_ids, max_new_tokens, eos_token_id, temperature, seed).request_id

    def request(self, request_id: int) -> GenerationRequest:
        try:
            return self.scheduler.requests[request_id]
        except KeyError:
            raise KeyError(f"request id not found: {request_id}") from None

    def finished(self, request_id: int) -> bool:
        return self.request(request_id).finished

    def generate_until_finished(self, request_id: int) -> List[int]:
        """Step until this request is finished (others in the queue advance too); returns prompt
        plus generated ids, like the reference (src/engine/paged_generate_engine.cpp:343-365)."""
        req = self.request(request_id)
        while not req.finished:
            self.step()
        return list(req.input_ids)

    def release_request(self, request_id: int) -> None:
        """Forget a request.  A finished request holds no pages (they went back when it
        finished); an unfinished one is taken out of the queues and its pages freed (a token of
        it that a launched step is still sampling is dropped when it arrives)."""
        req = self.request(request_id)
        if not req.finished:
            self.scheduler.release(req)
        del self.scheduler.requests[request_id]

    # ---- stepping --------------------------------------------------------------------------
    def _launch(self, plan: List[ScheduledPortion]):
        """Everything of a step that needs no answer from the device: pages, metadata, kernels,
        sampling into `runner.sampled`, and the start of the copy of the sampled tokens."""
        entries, samplers, admitted = [], [], []
        for p in plan:
            req, known = p.request, len(p.request.input_ids)
            if p.cached_len == 0:             # first portion since admission: bind its random stream (in this step's upload)
                admitted.append(("sampler", p.slot, slot_state_row(req.seed, len(req.generated_ids) + req.pending,
                                                                   req.temperature)))
            end = p.cached_len + p.num_tokens
            toks = req.input_ids[p.cached_len:end]
            feedback = -1
            if end > known:                   # the portion ends with the token that is still on the device
                toks = toks + [0]
                feedback = p.feedback_index
            entries.append(StepEntry(p.slot, toks, [p.num_tokens - 1] if p.samples else [], feedback=feedback))
            if p.samples:
                samplers.append(req)
        batch = self.runner.prepare(entries, state_writes=admitted)
        logits = self.runner.forward(batch)
        self.runner.finish(batch)
        which = self._launched & 1
        self._launched += 1
        if samplers:
            dev = self.sampler.sample(logits, batch.want_slot, any(r.temperature > 0 for r in samplers),
                                      out=self.runner.sampled[:len(samplers)])
            self._tokens_pinned[which][:len(samplers)].copy_(dev, non_blocking=True)
            self._read_done[which].record()
        if self.verbose:
            print(f"[step {self.runner.steps_run}] tokens={batch.num_tokens} entries={batch.num_entries}")
        return plan, samplers, which

    def _deliver(self, launched) -> List[tuple]:
        plan, samplers, which = launched
        tokens: List[int] = []
        if samplers:
            self._read_done[which].synchronize()
            tokens = self._tokens_pinned[which][:len(samplers)].tolist()
        out = [(r.request_id, t) for r, t in self.scheduler.deliver(plan, tokens)]
        if self.verbose and out:
            print(f"[tokens] {out}")
        return out

    def step(self) -> List[tuple]:
        """Launch one scheduled batch and return [(request id, token)] of the tokens that
        became known to the host in this call: this batch's own when not pipelined, the
        previous batch's when pipelined (an empty list at the very first step)."""
        plan = self.scheduler.schedule()
        launched = None
        if plan:
            launched = self._launch(plan)
            self.scheduler.advance(plan)
        if not self.pipelined:
            return self._deliver(launched) if launched else []
        before, self._in_flight = self._in_flight, launched
        return self._deliver(before) if before else []

    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._in_flight is not None

    def run(self) -> None:
        while self.has_work():
            self.step()
        self.runner.check_status()

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int, eos_token_id: int = -1,
                 temperature: float = 0.0, seed: int = 0) -> List[List[int]]:
        """Token ids in, new token ids out, for a list of prompts run together."""
        ids = [self.add_request(p, max_new_tokens, eos_token_id, temperature, seed + i)
               for i, p in enumerate(prompts)]
        self.run()
        out = [list(self.request(i).generated_ids) for i in ids]
        for i in ids:
            self.release_request(i)
        return out
