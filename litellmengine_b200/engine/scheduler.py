"""The scheduler: which requests run in the next step, and with how many tokens.

Pure host logic over the cache manager's bookkeeping, so its decisions are tested on the
CPU; the records and the decisions themselves are native code (`csrc/host_core.cpp`), this
class gives them their names and keeps the token lists.  The reference has no scheduler: it
prefills each prompt whole, one request at a time, then decodes all unfinished requests
together, and sizes the pool so that pages never run out
(src/engine/paged_generate_engine.cpp:343-365, src/benchmark/generation_benchmark.cpp:
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

import ctypes
from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np

from ..cache import CacheManager
from ..cache.pages import _check
from ..csrc import host
from .request import GenerationRequest

_SIGNATURES = {
    "hc_sched_new": ([ctypes.c_void_p, ctypes.c_longlong, ctypes.c_longlong], ctypes.c_void_p),
    "hc_sched_delete": ([ctypes.c_void_p], None),
    "hc_sched_add": ([ctypes.c_void_p, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_int, ctypes.POINTER(ctypes.c_int)], ctypes.c_int),
    "hc_sched_has_work": ([ctypes.c_void_p], ctypes.c_int),
    "hc_sched_num_preemptions": ([ctypes.c_void_p], ctypes.c_longlong),
    "hc_sched_queue": ([ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int], ctypes.c_int),
    "hc_sched_get": ([ctypes.c_void_p, ctypes.c_int, ctypes.c_int], ctypes.c_longlong),
    "hc_sched_schedule": ([ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                           ctypes.c_int, ctypes.POINTER(ctypes.c_int)], ctypes.c_int),
    "hc_sched_advance": ([ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int], None),
    "hc_sched_deliver": ([ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                          ctypes.c_void_p], ctypes.c_int),
    "hc_sched_release": ([ctypes.c_void_p, ctypes.c_int], ctypes.c_int),
}


def _library():
    lib = host.lib()
    if lib.hc_sched_new.argtypes is None:
        for name, (argtypes, restype) in _SIGNATURES.items():
            f = getattr(lib, name)
            f.argtypes, f.restype = argtypes, restype
    return lib


@dataclass
class ScheduledPortion:
    request: GenerationRequest
    num_tokens: int
    samples: bool          # the portion ends at the request's last token, so a token is sampled
    # the request's records when the plan was made (what the step's entry is built from)
    slot: int = -1
    cached_len: int = 0
    feedback_index: int = -1


class Scheduler:
    def __init__(self, cache: CacheManager, max_tokens_per_step: int = 8192, chunk: Optional[int] = None):
        if max_tokens_per_step <= 0:
            raise ValueError("max_tokens_per_step must be positive")
        self.cache = cache
        self.max_tokens_per_step = max_tokens_per_step
        self.chunk = min(chunk or max_tokens_per_step, max_tokens_per_step)
        if self.chunk <= 0:
            raise ValueError("chunk must be positive")
        self._lib = _library()
        self._h = self._lib.hc_sched_new(cache._h, max_tokens_per_step, self.chunk)
        if not self._h:
            raise ValueError(host.last_error())
        self.requests: Dict[int, GenerationRequest] = {}
        n = cache.max_slots
        self._ids = np.empty(n, np.int32)                  # the plan the native scheduler writes
        self._tokens = np.empty(n, np.int64)
        self._samples = np.empty(n, np.int32)
        self._admitted = np.empty(n, np.int32)
        self._facts = np.empty((n, 4), np.int64)

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.hc_sched_delete(self._h)
            self._h = None

    def _record(self, request_id: int, field: int) -> int:
        return self._lib.hc_sched_get(self._h, request_id, field)

    def _queue(self, which: int) -> List[GenerationRequest]:
        n = self._lib.hc_sched_queue(self._h, which, None, 0)
        ids = np.empty(n, np.int32)
        self._lib.hc_sched_queue(self._h, which, ids.ctypes.data, n)
        return [self.requests[i] for i in ids.tolist() if i in self.requests]

    @property
    def waiting(self) -> List[GenerationRequest]:
        """First come first served; a preempted request stands at the front.  A copy."""
        return self._queue(0)

    @property
    def running(self) -> List[GenerationRequest]:
        """In admission order.  A copy."""
        return self._queue(1)

    @property
    def num_preemptions(self) -> int:
        return self._lib.hc_sched_num_preemptions(self._h)

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
        rid = ctypes.c_int()
        _check(self._lib.hc_sched_add(self._h, len(prompt), int(max_new_tokens), int(eos_token_id), ctypes.byref(rid)))
        req = GenerationRequest(self._record, rid.value, prompt, int(max_new_tokens), int(eos_token_id),
                                float(temperature), int(seed))
        self.requests[req.request_id] = req
        return req

    def release(self, req: GenerationRequest) -> None:
        """Forget an unfinished request: out of the queues, its pages and slot freed (a token of it
        that a launched step is still sampling is dropped when it arrives)."""
        _check(self._lib.hc_sched_release(self._h, req.request_id))

    def has_work(self) -> bool:
        return bool(self._lib.hc_sched_has_work(self._h))

    # ---- one step --------------------------------------------------------------------------
    def schedule(self) -> List[ScheduledPortion]:
        count = ctypes.c_int()
        _check(self._lib.hc_sched_schedule(self._h, self._ids.ctypes.data, self._tokens.ctypes.data, self._samples.ctypes.data,
                                           self._admitted.ctypes.data, self._facts.ctypes.data, len(self._ids), ctypes.byref(count)))
        n = count.value
        plan = []
        for rid, tokens, samples, admitted, (slot, cached, _, fed) in zip(
                self._ids[:n].tolist(), self._tokens[:n].tolist(), self._samples[:n].tolist(), self._admitted[:n].tolist(),
                self._facts[:n].tolist()):
            if admitted:                                  # a slot taken just now: its state tensors start from zero
                for t in self.cache.state.values():
                    t[slot].zero_()
            plan.append(ScheduledPortion(self.requests[rid], tokens, bool(samples), slot, cached, fed))
        return plan

    def _plan_arrays(self, plan: List[ScheduledPortion]):
        ids = np.fromiter((p.request.request_id for p in plan), np.int32, len(plan))
        tokens = np.fromiter((p.num_tokens for p in plan), np.int64, len(plan))
        samples = np.fromiter((p.samples for p in plan), np.int32, len(plan))
        return ids, tokens, samples

    def advance(self, plan: List[ScheduledPortion]) -> None:
        """The step of `plan` has been launched: its tokens count as cached, and each portion
        that samples leaves a pending token (`feedback_index` = its place among the step's
        sampled tokens, in plan order)."""
        ids, tokens, samples = self._plan_arrays(plan)
        self._lib.hc_sched_advance(self._h, ids.ctypes.data, tokens.ctypes.data, samples.ctypes.data, len(plan))

    def deliver(self, plan: List[ScheduledPortion], sampled: List[int]) -> List[tuple]:
        """The host has read the tokens of the step of `plan` (one per portion with `samples`, in
        plan order): append them, free finished requests' pages and slots.  Returns
        [(request, token)] of the tokens that count; a token sampled for a request that had
        already finished (end of sequence found one step late, or released) is dropped."""
        ids, _, samples = self._plan_arrays(plan)
        toks = np.ascontiguousarray(sampled, dtype=np.int32)
        kept = np.zeros(len(toks), np.int32)
        _check(self._lib.hc_sched_deliver(self._h, ids.ctypes.data, samples.ctypes.data, len(plan), toks.ctypes.data, len(toks),
                                          kept.ctypes.data))
        out = []
        owners = [p.request for p in plan if p.samples]
        for req, token, keep in zip(owners, toks.tolist(), kept.tolist()):
            if keep:
                req.input_ids.append(token)
                req.generated_ids.append(token)
                out.append((req, token))
        return out

    def update(self, plan: List[ScheduledPortion], sampled: List[int]) -> List[GenerationRequest]:
        """After a step ran and its tokens were read: `advance` and `deliver` in one.  Returns the
        requests that finished."""
        self.advance(plan)
        return [r for r, _ in self.deliver(plan, sampled) if r.finished]
