from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, FeedForward,
                   GroupView, LayerCache, Mixer, Norm, OwedNorm, PagedKV, Part,
                   PositionEncoding, Registry, SlotState, StepContext, TensorSpec)

__all__ = [
    "BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "FeedForward",
    "GroupView", "LayerCache", "Mixer", "Norm", "OwedNorm", "PagedKV", "Part",
    "PositionEncoding", "Registry", "SlotState", "StepContext", "TensorSpec",
]
