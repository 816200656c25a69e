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
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import List, Optional


class RequestStatus(enum.Enum):
    WAITING = "waiting"          # not admitted (new, or preempted and to be recomputed)
    RUNNING = "running"          # holds a slot; prefilling while extend_len > 1 or nothing generated
    FINISHED = "finished"


@dataclass(eq=False)            # a request is itself: lists of requests are searched by identity
class GenerationRequest:
    request_id: int
    input_ids: List[int]
    prompt_len: int
    max_new_tokens: int
    eos_token_id: int = -1
    temperature: float = 0.0
    seed: int = 0
    generated_ids: List[int] = field(default_factory=list)
    cached_len: int = 0
    slot: int = -1
    status: RequestStatus = RequestStatus.WAITING
    preemptions: int = 0
    finish_reason: Optional[str] = None
    pending: int = 0             # sampled tokens of this request that are still on the device (1 when a step is planned)
    feedback_index: int = -1     # where among the last launched step's sampled tokens its token is

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

    def append_token(self, token: int) -> None:
        """src/engine/request_manager.cpp:122-159"""
        if self.status is RequestStatus.FINISHED:
            raise RuntimeError("append_token on a finished request")
        self.input_ids.append(int(token))
        self.generated_ids.append(int(token))
        if self.eos_token_id >= 0 and token == self.eos_token_id:
            self.status, self.finish_reason = RequestStatus.FINISHED, "eos"
        elif len(self.generated_ids) >= self.max_new_tokens:
            self.status, self.finish_reason = RequestStatus.FINISHED, "length"
