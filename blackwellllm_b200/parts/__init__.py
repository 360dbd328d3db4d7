"""Parts of a decoder: norms, position encodings, mixers, feed-forwards, blocks."""
from .base import (Block, BuildContext, FeedForward, FixedStateRequest, Mixer, Norm, PagedKVRequest,
                   ParamSpec, Part, PositionEncoding, build_block, build_ffn, build_mixer, build_norm,
                   build_position, register_block, register_ffn, register_mixer, register_norm,
                   register_position)
from . import attention, block, mlp, norm, rope  # noqa: F401  (registers the built-in parts)
from .linear import Linear
