from . import attention, block, embedding, mlp, norm, rope  # noqa: F401  (registers the built-in parts)
from .base import Block, FeedForward, Mixer, Norm, Part, PositionEncoding, Runtime, WeightSpec
from .registry import lookup, register, registered, unregister
from .spec import ExtraPart, LayerSpec, ModelSpec, PartSpec, ScheduleEntry

__all__ = ["Block", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "Runtime", "WeightSpec",
           "lookup", "register", "registered", "unregister", "ExtraPart", "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry"]
