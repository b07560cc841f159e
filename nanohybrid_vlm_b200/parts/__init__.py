from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401  (register the built-in parts)
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, Block, BuildEnv, CacheView, FeedForward,
                   FixedStateNeed, Mixer, Norm, PagedKVNeed, Part, PositionEncoding)
from .spec import LayerRun, LayerSpec, ModelSpec, ParamDecl, PartSpec, PartUse, Source, part

__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "Block", "BuildEnv", "CacheView", "FeedForward",
           "FixedStateNeed", "Mixer", "Norm", "PagedKVNeed", "Part", "PositionEncoding", "LayerRun", "LayerSpec",
           "ModelSpec", "ParamDecl", "PartSpec", "PartUse", "Source", "part"]
