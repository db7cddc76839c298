"""Parts that layers are put together from, and the records that describe a model."""
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, Block, CacheNeed, FeedForward, HeadPrep, HeadShape, Mixer,
                   Norm, Part, PartRegistry, Positions, StateNeed)
from .spec import (EmbeddingSpec, HeadSpec, LayerSpec, ModelSpec, PartSpec, ScheduleEntry,
                   default_schedule)
from .layout import expected_tensors
from . import (attention, block, feedforward, gla, latent_attention, matrix_memory, moe, norm, parallel,  # noqa: F401
               position, sigmoid_attention)  # noqa: F401  (register the built-in kinds)

__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "Block", "CacheNeed", "FeedForward",
           "HeadPrep", "HeadShape", "Mixer", "Norm", "Part", "PartRegistry", "Positions", "StateNeed", "EmbeddingSpec", "HeadSpec",
           "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "default_schedule", "expected_tensors"]
