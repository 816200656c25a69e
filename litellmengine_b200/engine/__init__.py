"""The engine: step batches, the step function, requests, the scheduler, generation."""
from .batch import StepBatch, StepBuffers, StepEntry
from .runner import ModelRunner

__all__ = ["StepBatch", "StepBuffers", "StepEntry", "ModelRunner"]
