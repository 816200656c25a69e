"""Picking next tokens: greedy argmax and temperature sampling, on the device.

The reference parses --temperature, --top-k and --top-p, warns that sampling is not
implemented and takes the argmax (src/main.cpp:175-178, src/runtime/args.cpp:101-106); ties
go to the lowest index (src/ops/argmax.cu:55,106-107).  Here temperature 0 is that argmax and
a positive temperature samples from softmax(logits / T); top-k and top-p are accepted by the
command line and, as in the reference, not applied.

Each request's random stream is part of its fixed-size state slot on the device:
int32 {seed low, seed high, counter, temperature bits}.  The u for a request's n-th sampled
token is a function of (seed, n) only.
"""
from __future__ import annotations

import struct
from typing import List

import torch

from ..csrc import ops


def slot_state_row(seed: int, counter: int, temperature: float) -> List[int]:
    """The four int32 of a request's stream, written into its slot by the step that admits it
    (counter = tokens it has sampled so far, so a recomputed request continues its own stream)."""
    seed &= 0xFFFFFFFFFFFFFFFF
    lo, hi = seed & 0xFFFFFFFF, seed >> 32
    tbits = struct.unpack("<i", struct.pack("<f", float(temperature)))[0]
    to_i32 = lambda v: v - (1 << 32) if v >= (1 << 31) else v
    return [to_i32(lo), to_i32(hi), to_i32(counter & 0xFFFFFFFF), tbits]


class Sampler:
    def __init__(self, sampler_state: torch.Tensor):
        self.state = sampler_state            # int32 [slots, 4] inside the cache manager's state slots

    def sample(self, logits: torch.Tensor, want_slot: torch.Tensor, any_sampling: bool,
               out: torch.Tensor = None) -> torch.Tensor:
        """int32 [rows] on the device (written into `out` when given)."""
        if not any_sampling:
            return ops.argmax_rows(logits, out=out)
        return ops.sample_rows(logits, want_slot, self.state, out=out)
