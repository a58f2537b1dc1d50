from .base import (ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, Arrangement, FeedForward,
                   FixedState, LayerCache, Mixer, Norm, PagedKV, Part, Position, Runtime, StepContext,
                   build_part, register_arrangement, register_feed_forward, register_mixer,
                   register_norm, register_position)
from .model import DecoderModel

__all__ = [
    "ARRANGEMENTS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "Arrangement", "FeedForward",
    "FixedState", "LayerCache", "Mixer", "Norm", "PagedKV", "Part", "Position", "Runtime",
    "StepContext", "build_part", "register_arrangement", "register_feed_forward", "register_mixer",
    "register_norm", "register_position", "DecoderModel",
]
