from . import attention, block, embedding, feedforward, norm, position  # noqa: F401 (register)
from .base import (
    Block,
    BuildEnv,
    CacheBinding,
    FeedForward,
    Mixer,
    Norm,
    PagedKVRequest,
    Part,
    PositionEncoding,
    StateRequest,
    WeightDecl,
)
from .registry import build_part, register_part, registered_kinds

__all__ = [
    "Block", "BuildEnv", "CacheBinding", "FeedForward", "Mixer", "Norm", "PagedKVRequest",
    "Part", "PositionEncoding", "StateRequest", "WeightDecl", "build_part", "register_part",
    "registered_kinds",
]
