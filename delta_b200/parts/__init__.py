"""Parts of a layer: norms, position encodings, mixers, feed-forwards, blocks."""
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, CacheSpec, FeedForward, Mixer, Norm,
                   Part, PartSpec, PositionEncoding, Registry, StateSpec, TensorSpec)
from . import (attention, block, decay_attention, experts, feed_forward, latent_attention, norm, residual, rope,  # noqa: F401
               row_attention, selective_scan, streams)  # (registers the parts)
