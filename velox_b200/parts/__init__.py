"""Parts a model is put together from.  Importing the package registers the built-in ones."""
from . import attention, block, io, mlp, norms, rope  # noqa: F401
from .base import (
    CacheNeeds,
    FeedForward,
    HiddenState,
    Mixer,
    Norm,
    PagedCacheSpec,
    Part,
    PositionEncoding,
    StateSpec,
)
from .registry import part_class, register_part, unregister_part
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSource, WeightSpec

__all__ = [
    "CacheNeeds", "FeedForward", "HiddenState", "LayerSpec", "Mixer", "ModelSpec", "Norm",
    "PagedCacheSpec", "Part", "PartSpec", "PositionEncoding", "ScheduleEntry", "StateSpec",
    "TensorSource", "WeightSpec", "part_class", "register_part", "unregister_part",
]
