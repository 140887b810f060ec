"""The step function and the generation loop."""

from .batch import StepBatch, StepLayout
from .runtime import Runtime, Workspace

__all__ = ["StepBatch", "StepLayout", "Runtime", "Workspace"]
