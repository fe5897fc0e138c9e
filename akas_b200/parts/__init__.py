"""Mixers, feed-forwards, norms, position encodings, and the block that arranges them."""

from .base import (
    FeedForward,
    Mixer,
    Normed,
    PagedKVSpec,
    PagedSpec,
    Param,
    Part,
    Runtime,
    StateSpec,
    build_part,
    project,
    project_swiglu,
    register_ffn,
    register_mixer,
    register_norm,
    register_position,
)
from .attention import Attention
from .block import ARRANGEMENTS, Block
from .norm import RMSNorm
from .rope import Rope
from .shortconv import ShortConv
from .swiglu import SwiGLU

__all__ = [
    "ARRANGEMENTS", "Attention", "Block", "FeedForward", "Mixer", "Normed", "PagedKVSpec", "PagedSpec", "Param", "Part", "RMSNorm",
    "Rope", "Runtime", "ShortConv", "StateSpec", "SwiGLU", "build_part", "project", "project_swiglu", "register_ffn", "register_mixer",
    "register_norm", "register_position",
]
