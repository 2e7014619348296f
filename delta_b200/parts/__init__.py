"""Parts of a layer: norms, position encodings, mixers, feed-forwards, blocks."""
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, CacheSpec, FeedForward, Mixer, Norm,
                   Part, PartSpec, PositionEncoding, Registry, StateSpec, TensorSpec)
from . import (attention, block, feed_forward, latent_attention, norm, rope, row_attention, selective_scan,  # noqa: F401
               streams)  # (registers the parts)
