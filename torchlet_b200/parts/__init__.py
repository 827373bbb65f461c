"""Parts a layer is put together from.  Importing this package registers the built-in
kinds; further kinds register themselves with the same decorators."""
from .base import (
    BLOCKS,
    FEED_FORWARDS,
    MIXERS,
    NORMS,
    POSITIONS,
    Block,
    FeedForward,
    KVSpec,
    Mixer,
    Norm,
    Part,
    Positions,
    StateSpec,
    TensorSpec,
    build_part,
)
from . import attention, block, norm, rotary, swiglu  # noqa: F401  (registration)
from .linear import Linear
from .model import LayeredModel, expected_tensors

__all__ = [
    "BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "Block", "FeedForward", "KVSpec",
    "LayeredModel", "Linear", "Mixer", "Norm", "Part", "Positions", "StateSpec", "TensorSpec",
    "build_part", "expected_tensors",
]
