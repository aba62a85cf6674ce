"""Parts a layer is put together from: mixer, feed-forward, norm, position encoding, block."""

from . import (attention, biased_attention, block, delta_rule, feed_forward,  # noqa: F401
               general_delta, latent_attention, norm, normed_attention, position, routed,
               side_by_side, stream_join,
               token_shift, token_side)  # (registration)
from .base import (Block, BuildContext, CacheView, FeedForward, KVSpec, Mixer, Norm, Part,
                   PositionEncoding, SideInput, StateSpec, StreamJoin, TokenMix)
from .registry import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, SIDE_INPUTS,
                       STREAM_JOINS, TOKEN_MIXES, make, register_stream_join, register_token_mix,
                       register_block, register_feed_forward, register_mixer, register_norm,
                       register_position_encoding, register_side_input)

__all__ = ["BLOCKS", "Block", "BuildContext", "CacheView", "FEED_FORWARDS", "FeedForward", "KVSpec",
           "MIXERS", "Mixer", "NORMS", "Norm", "POSITION_ENCODINGS", "Part",
           "PositionEncoding", "SIDE_INPUTS", "STREAM_JOINS", "SideInput", "StateSpec", "StreamJoin",
           "TOKEN_MIXES", "TokenMix", "register_stream_join",
           "register_token_mix", "make", "register_side_input", "register_block", "register_feed_forward",
           "register_mixer", "register_norm", "register_position_encoding"]
