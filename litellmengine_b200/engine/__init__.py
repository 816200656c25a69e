"""The engine: step batches, the step function, requests, the scheduler, generation."""
from .batch import StepBatch, StepBuffers, StepEntry
from .request import GenerationRequest, RequestStatus
from .scheduler import ScheduledPortion, Scheduler
from .runner import ModelRunner
from .generate import PagedGenerateEngine

__all__ = ["StepBatch", "StepBuffers", "StepEntry", "GenerationRequest", "RequestStatus",
           "ScheduledPortion", "Scheduler", "ModelRunner", "PagedGenerateEngine"]
