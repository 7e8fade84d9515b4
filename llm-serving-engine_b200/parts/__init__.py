"""Parts a model is assembled from. Importing this package registers the built-in kinds."""

from . import attention, blocks, feed_forward, norms, positions  # noqa: F401
from .attention import AttentionSpec, PagedAttention
from .base import (
    BLOCKS,
    FEED_FORWARDS,
    MIXERS,
    NORMS,
    POSITION_ENCODINGS,
    Block,
    BuildEnv,
    FeedForward,
    Mixer,
    Norm,
    PagedKVNeed,
    ParamDecl,
    Part,
    PositionEncoding,
    StateNeed,
    role_dtype,
)
from .blocks import PreNormBlock, PreNormBlockSpec
from .feed_forward import SwiGLU, SwiGLUSpec
from .norms import RMSNorm, RMSNormSpec
from .positions import NoPositionSpec, RotaryPositionEncoding, RotarySpec

__all__ = [
    "AttentionSpec", "PagedAttention", "BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS",
    "POSITION_ENCODINGS", "Block", "BuildEnv", "FeedForward", "Mixer", "Norm", "PagedKVNeed",
    "ParamDecl", "Part", "PositionEncoding", "StateNeed", "role_dtype", "PreNormBlock",
    "PreNormBlockSpec", "SwiGLU", "SwiGLUSpec", "RMSNorm", "RMSNormSpec", "NoPositionSpec",
    "RotaryPositionEncoding", "RotarySpec",
]
