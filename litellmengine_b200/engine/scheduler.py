"""The scheduler: which requests run in the next step, and with how many tokens.

Pure host logic over the cache manager's bookkeeping, so its decisions are tested on the
CPU.  The reference has no scheduler: it prefills each prompt whole, one request at a time,
then decodes all unfinished requests together, and sizes the pool so that pages never run
out (src/engine/paged_generate_engine.cpp:343-365, src/benchmark/generation_benchmark.cpp:
152-159,291-315); when they do run out it throws (src/engine/block_table_manager.cpp:82-84).

Rules, in this order, every step:
  1. Running requests that decode (one new token each) go first, oldest admission first.
  2. Running requests still reading their prompt get a portion of at most `chunk` tokens,
     limited by what is left of `max_tokens_per_step`.
  3. Waiting requests are admitted first-come first-served while a slot is free, budget is
     left and the pages of their first portion are free; admission stops at the first one
     that does not fit (no overtaking).
  When pages run out for a running request (1 or 2), the most recently admitted running
  request is preempted: its pages and slot are given back, its tokens are kept, and it goes
  to the FRONT of the waiting queue to be recomputed from its first token.  This repeats
  until the older request fits; a request alone always fits because `add` refuses requests
  longer than the pool.  All choices depend only on the order of `add` calls.

A step's result may be read one step late: `advance(plan)` books a launched step (lengths move
on, each sampled token is `pending`), `deliver(plan, tokens)` books its tokens when the host has
them; `update` is both at once.  Between the two, `schedule` already plans the next step: a
request whose pending token is its last (by `max_new_tokens`) is left out, one that turns out
to have ended with its end-of-sequence token has run one token too many, which `deliver` drops.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass
from typing import Deque, Dict, List, Optional

from ..cache import CacheManager, OutOfPages
from .request import GenerationRequest, RequestStatus


@dataclass
class ScheduledPortion:
    request: GenerationRequest
    num_tokens: int
    samples: bool          # the portion ends at the request's last token, so a token is sampled


class Scheduler:
    def __init__(self, cache: CacheManager, max_tokens_per_step: int = 8192, chunk: Optional[int] = None):
        if max_tokens_per_step <= 0:
            raise ValueError("max_tokens_per_step must be positive")
        self.cache = cache
        self.max_tokens_per_step = max_tokens_per_step
        self.chunk = min(chunk or max_tokens_per_step, max_tokens_per_step)
        if self.chunk <= 0:
            raise ValueError("chunk must be positive")
        self.waiting: Deque[GenerationRequest] = deque()
        self.running: List[GenerationRequest] = []       # in admission order
        self.requests: Dict[int, GenerationRequest] = {}
        self._next_id = 0
        self.num_preemptions = 0

    # ---- requests --------------------------------------------------------------------------
    def add(self, prompt_ids, max_new_tokens: int, eos_token_id: int = -1, temperature: float = 0.0,
            seed: int = 0) -> GenerationRequest:
        prompt = [int(t) for t in prompt_ids]
        if not prompt:
            raise ValueError("a request needs at least one prompt token")
        if max_new_tokens < 0:
            raise ValueError("max_new_tokens must be >= 0")
        if temperature < 0:
            raise ValueError("--temperature must be >= 0")
        # the last sampled token is never run, so the cache holds at most prompt + new - 1
        longest = len(prompt) + max(max_new_tokens - 1, 0)
        if longest > self.cache.max_request_tokens:
            raise OutOfPages(f"request needs {longest} cached tokens; the cache takes at most "
                             f"{self.cache.max_request_tokens} per request")
        req = GenerationRequest(self._next_id, prompt, len(prompt), max_new_tokens, eos_token_id,
                                float(temperature), int(seed))
        self._next_id += 1
        self.requests[req.request_id] = req
        if max_new_tokens == 0:
            req.status, req.finish_reason = RequestStatus.FINISHED, "length"
        else:
            self.waiting.append(req)
        return req

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- one step --------------------------------------------------------------------------
    def _preempt_latest(self) -> GenerationRequest:
        victim = self.running.pop()
        self.cache.release(victim.slot)
        victim.slot, victim.cached_len = -1, 0
        victim.status = RequestStatus.WAITING
        victim.preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(victim)
        return victim

    def schedule(self) -> List[ScheduledPortion]:
        budget = self.max_tokens_per_step
        plan: List[ScheduledPortion] = []
        need = [0] * len(self.cache.groups)               # pages per group already promised in this step

        preempted = False
        i = 0
        order = sorted(range(len(self.running)), key=lambda k: (self.running[k].extend_len > 1, k))
        queue = [self.running[k] for k in order]          # decoders first, each kind oldest first
        while i < len(queue):
            req = queue[i]
            if req.status is not RequestStatus.RUNNING or req.remain_len <= 0:   # preempted below, or only awaiting its last token
                i += 1
                continue
            if budget <= 0:
                break
            n = min(req.extend_len, self.chunk, budget)
            while True:
                got = self.cache.reserve(need, req.slot, req.cached_len + n)
                if got is not None:
                    break
                victim = self._preempt_latest()
                preempted = True
                plan = [p for p in plan if p.request is not victim]
                budget = self.max_tokens_per_step - sum(p.num_tokens for p in plan)
                need = [0] * len(self.cache.groups)
                for p in plan:                            # the pool changed: count the promises again
                    need = self.cache.reserve(need, p.request.slot, p.request.cached_len + p.num_tokens)
                if victim is req:
                    break
            if req.status is not RequestStatus.RUNNING:
                i += 1
                continue
            need = got
            plan.append(ScheduledPortion(req, n, n == req.extend_len))
            budget -= n
            i += 1

        # no admission in a step that had to preempt: the victim would come straight back
        while not preempted and self.waiting and budget > 0 and self.cache.free_slots > 0:
            req = self.waiting[0]
            if req.remain_len <= 0:                       # preempted with its last token on its way
                break
            n = min(req.extend_len, self.chunk, budget)
            got = self.cache.reserve(need, None, n)
            if got is None:
                break
            need = got
            self.waiting.popleft()
            req.slot = self.cache.admit()
            req.status = RequestStatus.RUNNING
            self.running.append(req)
            plan.append(ScheduledPortion(req, n, n == req.extend_len))
            budget -= n
        if not plan and self.has_work() and not any(r.pending for r in list(self.running) + list(self.waiting)):
            raise OutOfPages("nothing can be scheduled: the cache is too small for the oldest request")
        return plan

    def advance(self, plan: List[ScheduledPortion]) -> None:
        """The step of `plan` has been launched: its tokens count as cached, and each portion
        that samples leaves a pending token (`feedback_index` = its place among the step's
        sampled tokens, in plan order)."""
        k = 0
        for p in plan:
            req = p.request
            req.cached_len += p.num_tokens
            if p.samples:
                req.pending += 1                          # two for a moment: the step before is read after this
                req.feedback_index = k
                k += 1

    def deliver(self, plan: List[ScheduledPortion], sampled: List[int]) -> List[tuple]:
        """The host has read the tokens of the step of `plan` (one per portion with `samples`, in
        plan order): append them, free finished requests' pages and slots.  Returns
        [(request, token)] of the tokens that count; a token sampled for a request that had
        already finished (end of sequence found one step late, or released) is dropped."""
        it = iter(sampled)
        out = []
        for p in plan:
            if not p.samples:
                continue
            req, token = p.request, next(it)
            req.pending -= 1
            if req.finished:
                continue
            req.append_token(token)
            out.append((req, token))
            if req.finished:
                if req in self.running:
                    self.running.remove(req)
                    self.cache.release(req.slot)
                    req.slot = -1
                elif req in self.waiting:                 # preempted while its last token was on its way
                    self.waiting.remove(req)
        return out

    def update(self, plan: List[ScheduledPortion], sampled: List[int]) -> List[GenerationRequest]:
        """After a step ran and its tokens were read: `advance` and `deliver` in one.  Returns the
        requests that finished."""
        self.advance(plan)
        return [r for r, _ in self.deliver(plan, sampled) if r.finished]
