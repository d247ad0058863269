"""Layer parts: mixers, feed-forwards, norms, position encodings, block arrangements."""
from .base import (FeedForward, Mixer, Norm, PagedNeed, ParamDecl, Part, Position, StateNeed, StreamPart)
from .registry import (build_block, build_feed_forward, build_mixer, build_norm, build_position, build_stream,
                       register_block, register_feed_forward, register_mixer, register_norm,
                       register_position, register_stream, registered, unregister)
from . import (attention, block, feed_forward, gla, latent_attention, lightning, norm, rope, routed_experts,  # noqa: F401
               short_conv, sigmoid_attention, stream)  # noqa: F401  (register the built-in parts)

__all__ = [
    "FeedForward", "Mixer", "Norm", "PagedNeed", "ParamDecl", "Part", "Position", "StateNeed", "StreamPart",
    "build_block", "build_feed_forward", "build_mixer", "build_norm", "build_position", "build_stream",
    "register_block", "register_feed_forward", "register_mixer", "register_norm",
    "register_position", "register_stream", "registered", "unregister",
]
