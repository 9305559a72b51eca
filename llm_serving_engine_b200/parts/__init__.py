from . import attention, block, mlp, norm, rope  # noqa: F401  (register the built-in parts)
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, BuildContext,
                   FeedForward, Mixer, Norm, PagedKV, Part, PositionEncoding, RequestState,
                   ResidualStream, register_block, register_feed_forward, register_mixer,
                   register_norm, register_position_encoding)
from .linear import linear, linear_partials, reduce_partials

__all__ = [
    "BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Block", "BuildContext",
    "FeedForward", "Mixer", "Norm", "PagedKV", "Part", "PositionEncoding", "RequestState",
    "ResidualStream", "linear", "linear_partials", "reduce_partials", "register_block", "register_feed_forward", "register_mixer",
    "register_norm", "register_position_encoding",
]
