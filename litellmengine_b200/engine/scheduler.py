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
        reserved: List[tuple] = []         # (slot, new_len) already promised pages in this step

        def fits(slot, new_len) -> bool:
            return self.cache.can_hold(reserved + [(slot, new_len)])

        preempted = False
        i = 0
        order = sorted(range(len(self.running)), key=lambda k: (self.running[k].extend_len > 1, k))
        queue = [self.running[k] for k in order]          # decoders first, each kind oldest first
        while i < len(queue):
            req = queue[i]
            if req not in self.running:                   # preempted below
                i += 1
                continue
            if budget <= 0:
                break
            n = min(req.extend_len, self.chunk, budget)
            while not fits(req.slot, req.cached_len + n):
                victim = self._preempt_latest()
                preempted = True
                plan = [p for p in plan if p.request is not victim]
                reserved = [(p.request.slot, p.request.cached_len + p.num_tokens) for p in plan]
                budget = self.max_tokens_per_step - sum(p.num_tokens for p in plan)
                if victim is req:
                    break
            if req not in self.running:
                i += 1
                continue
            plan.append(ScheduledPortion(req, n, n == req.extend_len))
            reserved.append((req.slot, req.cached_len + n))
            budget -= n
            i += 1

        # no admission in a step that had to preempt: the victim would come straight back
        while not preempted and self.waiting and budget > 0 and self.cache.free_slots > 0:
            req = self.waiting[0]
            n = min(req.extend_len, self.chunk, budget)
            if not self.cache.can_hold(reserved + [(None, n)]):
                break
            self.waiting.popleft()
            req.slot = self.cache.admit()
            req.status = RequestStatus.RUNNING
            self.running.append(req)
            plan.append(ScheduledPortion(req, n, n == req.extend_len))
            reserved.append((req.slot, n))
            budget -= n
        if not plan and self.has_work():
            raise OutOfPages("nothing can be scheduled: the cache is too small for the oldest request")
        return plan

    def update(self, plan: List[ScheduledPortion], sampled: List[int]) -> List[GenerationRequest]:
        """After the step ran: advance cached lengths, append the sampled tokens (one per
        portion with `samples`, in plan order), free finished requests' pages and slots.
        Returns the requests that finished."""
        it = iter(sampled)
        done = []
        for p in plan:
            req = p.request
            req.cached_len += p.num_tokens
            if p.samples:
                req.append_token(next(it))
                if req.finished:
                    self.running.remove(req)
                    self.cache.release(req.slot)
                    req.slot = -1
                    done.append(req)
        return done
