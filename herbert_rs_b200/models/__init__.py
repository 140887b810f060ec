"""Models: the generic decoder, and the architectures registered for it."""

from ..config.qwen3 import Qwen3Config
from ..registry import register_architecture
from .decoder import DecoderModel

# "qwen3" is the reference's family key (crates/core/src/config.rs:93-103).
register_architecture("Qwen3ForCausalLM", Qwen3Config, model_types=("qwen3",), default=True)

__all__ = ["DecoderModel"]
