"""Parts that layers are put together from, and the records that describe a model."""
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, Block, CacheNeed, FeedForward, HeadShape, Mixer,
                   Norm, Part, PartRegistry, Positions, StateNeed)
from .spec import (EmbeddingSpec, HeadSpec, LayerSpec, ModelSpec, PartSpec, ScheduleEntry,
                   default_schedule)
from .layout import expected_tensors
from . import attention, block, feedforward, norm, position  # noqa: F401  (register the built-in kinds)

__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "Block", "CacheNeed", "FeedForward",
           "HeadShape", "Mixer", "Norm", "Part", "PartRegistry", "Positions", "StateNeed", "EmbeddingSpec", "HeadSpec",
           "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "default_schedule", "expected_tensors"]
