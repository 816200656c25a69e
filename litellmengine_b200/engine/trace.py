"""Trace replay: drive the step function with given tokens, step by step, and hand back logits.

This is the whole logic of `bin/trace_run`; it samples nothing and has no model, cache or
loader of its own — it admits a request when its id first appears, calls `ModelRunner.step`
with the step's entries as one batch, and releases the requests an `end` list names.
"""
from __future__ import annotations

from typing import Callable, Dict, Iterable, Optional

import torch

from .batch import StepEntry
from .runner import ModelRunner


def replay(runner: ModelRunner, steps: Iterable[dict],
           on_logits: Callable[[int, torch.Tensor], None],
           on_done: Optional[Callable[[int], None]] = None) -> None:
    """steps: dicts {"step": n, "entries": [{"id", "tokens", "want"}], "end": [ids]}.
    on_logits(step, float32 [wanted, vocab] on the device) is called for steps that want
    something; on_done(step) after every step."""
    slots: Dict[object, int] = {}
    for rec in steps:
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if rid not in slots:
                slots[rid] = runner.admit()
            entries.append(StepEntry(slots[rid], [int(t) for t in e["tokens"]],
                                     [int(w) for w in e.get("want", [])]))
        if entries:
            logits = runner.step(entries)
            if logits.shape[0]:
                on_logits(step, logits)
            runner.check_status()
        for rid in rec.get("end", []):
            if rid in slots:
                runner.release(slots.pop(rid))
        if on_done is not None:
            on_done(step)
