from . import attention, block, feed_forward, norm, position  # noqa: F401  (register the built-in kinds)
from .base import (BuildContext, FixedStateNeed, PagedKVNeed, PagedLayerCache, Part, StateLayerCache, StepContext,
                   TensorSpec)
from .model import Model
from .registry import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, register_block, register_feed_forward,
                       register_mixer, register_norm, register_position)

__all__ = ["BuildContext", "FixedStateNeed", "PagedKVNeed", "PagedLayerCache", "Part", "StateLayerCache",
           "StepContext", "TensorSpec", "Model", "BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS",
           "register_block", "register_feed_forward", "register_mixer", "register_norm", "register_position"]
