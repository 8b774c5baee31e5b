from . import (attention, block, connection, diff_attention, feedforward, latent_attention, lightning,  # noqa: F401
               mamba2, norm, rope, shared_kv_attention, transforms)      # (registers the built-in kinds)
from .base import (Connection, FeedForward, KVSpec, LayerSpec, Mixer, ModelSpec, Norm, Part, PartSpec,
                   PositionEncoding, ScheduleEntry, StateSpec, make_part, register_part,
                   registered_parts)

__all__ = [
    "Connection", "FeedForward", "KVSpec", "LayerSpec", "Mixer", "ModelSpec", "Norm", "Part", "PartSpec",
    "PositionEncoding", "ScheduleEntry", "StateSpec", "make_part", "register_part", "registered_parts",
]
