"""Parts a layer is put together from.  Importing this package registers the built-in ones."""
from . import (attention, block, embedding, gated_state, latent_attention, linear_attention, mlp, norm, rope, routed_mlp,  # noqa: F401  (registration)
               stream)
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, STREAM_STEPS, Block, BuildEnv,
                   FeedForward, LayerCache, Mixer, Norm, PagedCacheSpec, ParamSpec, Part, PositionEncoding, StateSpec,
                   StepContext, StreamStep, build_part)

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITIONS", "STREAM_STEPS", "StreamStep", "Block", "BuildEnv",
           "FeedForward", "LayerCache", "Mixer", "Norm", "PagedCacheSpec", "ParamSpec", "Part", "PositionEncoding",
           "StateSpec", "StepContext", "build_part"]
