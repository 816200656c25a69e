"""Parts a model is assembled from, and the model that runs them."""
from . import norms, position, attention, feed_forward, block     # registers the built-in kinds
from .registry import (lookup, register_arrangement, register_feed_forward, register_mixer,
                       register_norm, register_position, unregister)
from .context import StageContext, StepFacts, StepPrelude
from .position import Rotation
from .block import Block
from .model import Model, build_model, model_parameters

__all__ = ["lookup", "register_arrangement", "register_feed_forward", "register_mixer", "register_norm",
           "register_position", "unregister", "StageContext", "StepFacts", "StepPrelude", "Rotation", "Block", "Model", "build_model",
           "model_parameters"]
