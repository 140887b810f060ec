"""Parts of a layer.  Importing this package registers the built-in kinds."""

from .base import Block, FeedForward, Mixer, Norm, ParamSpec, Part
from .norm import RMSNorm
from .rope import RotaryEncoding, rope_tables
from .attention import AttentionMixer
from .swiglu import SwiGLU, join_gate_up
from .block import PreNormBlock

__all__ = ["Block", "FeedForward", "Mixer", "Norm", "ParamSpec", "Part", "RMSNorm", "RotaryEncoding",
           "rope_tables", "AttentionMixer", "SwiGLU", "join_gate_up", "PreNormBlock"]
