from . import (attention, block, connection, diff_attention, feedforward, lightning, norm, rope,  # noqa: F401
               transforms)      # (registers the built-in kinds)
from .base import (Connection, FeedForward, KVSpec, LayerSpec, Mixer, ModelSpec, Norm, Part, PartSpec,
                   PositionEncoding, ScheduleEntry, StateSpec, make_part, register_part,
                   registered_parts)

__all__ = [
    "Connection", "FeedForward", "KVSpec", "LayerSpec", "Mixer", "ModelSpec", "Norm", "Part", "PartSpec",
    "PositionEncoding", "ScheduleEntry", "StateSpec", "make_part", "register_part", "registered_parts",
]
