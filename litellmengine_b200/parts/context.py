"""What a mixer sees of the step it runs in."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

import torch


@dataclass
class StageContext:
    """The step's batch plus this stage's share of the cache.

    batch        the step's `StepBatch`: device arrays token_ids / positions / token_entry
                 [T], entry_slot / entry_q_start / entry_q_len / entry_kv_len [B], and the
                 same facts as host lists in `batch.entries`.
    stage        index of this stage in the model's run order.
    cache        [pages, 2, kv_heads, page_size, head_dim] of this stage (or of the stage it
                 borrows from), None if the stage's mixer asked for no pages.
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
