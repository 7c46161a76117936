from . import attention, block, embedding, mlp, norm, rope  # noqa: F401  (registers the built-in parts)
from .base import (Arrangement, Embedding, FeedForward, Head, Mixer, Norm, Part, PositionEncoding,
                   RotaryTable, Runtime)
from .registry import find_part, register_part, registered
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec

__all__ = ["Arrangement", "Embedding", "FeedForward", "Head", "Mixer", "Norm", "Part", "PositionEncoding",
           "RotaryTable", "Runtime", "find_part", "register_part", "registered", "LayerSpec", "ModelSpec",
           "PartSpec", "ScheduleEntry", "TensorSpec"]
