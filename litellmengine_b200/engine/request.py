"""Host records of generation requests and their state machine.

Fields and rules follow the reference's GenerationRequest / RequestManager
(include/engine/request.hpp:11-106, src/engine/request_manager.cpp:9-282): `input_ids` is
prompt plus generated tokens; `cached_len` counts tokens whose keys and values are in the
cache; a sampled token equal to `eos_token_id` (when >= 0) finishes the request and is kept;
so does reaching `max_new_tokens`; `max_new_tokens == 0` is finished at once.  Added: the
`Waiting` state covers both a request never run and one preempted (its pages were taken
away, its tokens kept), and a request may be prefilled in portions.  `pending` counts a
token that a launched step has sampled on the device and the host has not read yet: it is
part of the request's length (the next step may already run it) but not of `input_ids`.

The token lists and the request's facts live here; its lengths and states are the native
scheduler's records (`csrc/host_core.cpp`), read through it.
"""
from __future__ import annotations

import enum
from typing import List, Optional


class RequestStatus(enum.Enum):
    WAITING = "waiting"          # not admitted (new, or preempted and to be recomputed)
    RUNNING = "running"          # holds a slot; prefilling while extend_len > 1 or nothing generated
    FINISHED = "finished"


_STATUS = (RequestStatus.WAITING, RequestStatus.RUNNING, RequestStatus.FINISHED)
_FINISH = (None, "eos", "length", "released")
# field numbers of the native record
_F_STATUS, _F_SLOT, _F_PENDING, _F_FEEDBACK, _F_PREEMPTIONS, _F_FINISH, _F_CACHED = range(7)


class GenerationRequest:
    """A request is itself: lists of requests are searched by identity."""

    def __init__(self, records, request_id: int, prompt: List[int], max_new_tokens: int, eos_token_id: int = -1,
                 temperature: float = 0.0, seed: int = 0):
        self._get = records                  # (request id, field) -> the native record's value
        self.request_id = request_id
        self.input_ids = prompt
        self.prompt_len = len(prompt)
        self.max_new_tokens = max_new_tokens
        self.eos_token_id = eos_token_id
        self.temperature = temperature
        self.seed = seed
        self.generated_ids: List[int] = []

    status = property(lambda self: _STATUS[self._get(self.request_id, _F_STATUS)])
    slot = property(lambda self: self._get(self.request_id, _F_SLOT))
    cached_len = property(lambda self: self._get(self.request_id, _F_CACHED))
    preemptions = property(lambda self: self._get(self.request_id, _F_PREEMPTIONS))
    finish_reason = property(lambda self: _FINISH[self._get(self.request_id, _F_FINISH)])
    # sampled tokens of this request that are still on the device (1 when a step is planned)
    pending = property(lambda self: self._get(self.request_id, _F_PENDING))
    # where among the last launched step's sampled tokens its token is
    feedback_index = property(lambda self: self._get(self.request_id, _F_FEEDBACK))

    @property
    def device_len(self) -> int:
        """Tokens that have to be in the cache before the next token can be sampled."""
        return len(self.input_ids) + self.pending

    @property
    def extend_len(self) -> int:
        return len(self.input_ids) + self.pending - self.cached_len

    @property
    def remain_len(self) -> int:
        """Tokens still to be sampled by steps not yet launched."""
        return self.max_new_tokens - len(self.generated_ids) - self.pending

    @property
    def finished(self) -> bool:
        return self.status is RequestStatus.FINISHED

    def __repr__(self) -> str:
        return (f"GenerationRequest({self.request_id}, {self.status.value}, prompt {self.prompt_len}, "
                f"generated {len(self.generated_ids)}/{self.max_new_tokens}, cached {self.cached_len})")
