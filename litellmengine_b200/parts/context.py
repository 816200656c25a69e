"""What a mixer sees of the step it runs in."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional

import numpy as np
import torch


@dataclass
class StepFacts:
    """Per-entry facts of a step as numpy arrays, in entry order (what a prelude reads)."""
    q_start: np.ndarray      # first row of the entry in the batch
    q_len: np.ndarray        # tokens it brings
    past: np.ndarray         # tokens already cached
    slot: np.ndarray
    num_tokens: int


class StepPrelude:
    """What a part computes from a step's entries once, before any layer runs: work lists for its
    kernels (which rows go to which kernel, tiles, sorted orders).  The step function gives it room
    in the step's one pinned buffer, so its words travel to the device in the step's one copy.

    name                      key in `batch.preludes`; parts that offer a prelude of the same name share it.
    sections(tokens, entries) {section name: int32 words} it needs for a step of at most so many tokens
                              in so many entries.
    fill(facts, out)          write the words (`out`: {section name: numpy int32 view of the pinned
                              buffer}) from `facts` (a `StepFacts`); return whatever host-side facts
                              `views` needs.
    views(dev, filled)        the object kernels are launched from: device views into `dev` ({section
                              name: int32 device tensor at an address that is fixed per layout}) plus
                              host counts.
    """
    name = "prelude"

    def sections(self, max_tokens: int, max_entries: int) -> Dict[str, int]:
        raise NotImplementedError

    def fill(self, facts: StepFacts, out: Dict[str, np.ndarray]):
        raise NotImplementedError

    def views(self, dev: Dict[str, torch.Tensor], filled):
        raise NotImplementedError


@dataclass
class StageContext:
    """The step's batch plus this stage's share of the cache.

    batch        the step's `StepBatch`: device arrays token_ids / positions / token_entry
                 [T], entry_slot / entry_q_start / entry_q_len / entry_kv_len [B], and the
                 same facts as host lists in `batch.entries`.
    stage        index of this stage in the model's run order.
    cache        [pages, 2, kv_heads, page_size, head_dim] of this stage (or of the stage it
                 borrows from); None if the stage's mixer asked for no pages, or for keys and
                 values of different widths.
    cache_keys   [pages, kv_heads, page_size, key width] and
    cache_values [pages, kv_heads, page_size, value width] of the same pages (views of `cache`
                 when that exists, tensors of their own otherwise).
    block_table  device int32 [slots, pages per request] of the cache's group.
    writes_cache False when the cache belongs to another stage.
    state        [slots, *shape] tensor if the mixer asked for fixed-size state, else None.
    status       device int32 [2] where kernels record a refused index instead of trapping.
    partials_ok  True when whoever consumes the mixer's output adds up an `ops.PartialSum`
                 itself, so the mixer may return one instead of a tensor.
    residual     the float32 residual stream [T, hidden] that the mixer's result is about to be
                 added to, if the arrangement offers it: a mixer may add its result there itself
                 (in the epilogue of its last product) and return None.
    """
    batch: Any
    stage: int
    cache: Optional[torch.Tensor]
    block_table: Optional[torch.Tensor]
    page_size: int
    writes_cache: bool
    state: Optional[torch.Tensor]
    status: torch.Tensor
    partials_ok: bool = False
    residual: Optional[torch.Tensor] = None
    cache_keys: Optional[torch.Tensor] = None
    cache_values: Optional[torch.Tensor] = None
