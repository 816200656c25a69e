"""Sampling: greedy and temperature, with per-request random streams in the state slots."""
from .sampler import Sampler, slot_state_row

__all__ = ["Sampler", "slot_state_row"]
