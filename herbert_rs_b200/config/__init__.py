"""Typed configurations and the specs that parts are built from."""

from .base import Reader, read_config_json
from .qwen3 import Qwen3Config
from .specs import (AttentionSpec, BlockSpec, ModelSpec, NormSpec, PositionSpec,
                    ScheduleStep, SwiGLUSpec, identity_schedule)

__all__ = [
    "Reader", "read_config_json", "Qwen3Config", "AttentionSpec", "BlockSpec", "ModelSpec",
    "NormSpec", "PositionSpec", "ScheduleStep", "SwiGLUSpec", "identity_schedule",
]
