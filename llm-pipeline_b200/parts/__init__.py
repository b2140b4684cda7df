"""Parts: norm, position encoding, mixer, feed-forward, embedding, head, block arrangement."""

from .base import (Block, DepthMix, Embedding, FeedForward, Head, LayerCache, Mixer, Norm, Part, PositionEncoding,
                   ResidualStream)
from .registry import (kinds, lookup, register_block, register_depth_mix, register_embedding, register_feed_forward, register_head,
                       register_mixer, register_norm, register_position)
from . import (attention, block, capped_attention, delta_rule, depth_mix, differential_attention, embedding, experts, feed_forward,  # noqa: F401
               latent_attention, norm, position, recurrent, selective_scan, side_by_side, sigmoid_attention, state_space)  # noqa: F401  (register the built-in kinds)

__all__ = ["Block", "DepthMix", "Embedding", "FeedForward", "Head", "LayerCache", "Mixer", "Norm", "Part", "PositionEncoding",
           "ResidualStream", "kinds", "lookup", "register_block", "register_depth_mix", "register_embedding", "register_feed_forward",
           "register_head", "register_mixer", "register_norm", "register_position"]
