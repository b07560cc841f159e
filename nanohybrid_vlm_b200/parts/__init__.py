from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401  (register the built-in parts)
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, Block, BuildEnv, CacheView, Embedding,
                   FeedForward, FixedStateNeed, Head, Mixer, Norm, PagedKVNeed, Part, PositionEncoding)
from .spec import LayerRun, LayerSpec, ModelSpec, ParamDecl, PartSpec, PartUse, Source, part

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITIONS", "Block", "BuildEnv", "CacheView",
           "Embedding", "FeedForward", "FixedStateNeed", "Head", "Mixer", "Norm", "PagedKVNeed", "Part", "PositionEncoding",
           "LayerRun", "LayerSpec", "ModelSpec", "ParamDecl", "PartSpec", "PartUse", "Source", "part"]
