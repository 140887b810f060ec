"""Interfaces of the parts a layer is put together from.

A part is built from a spec (sizes and constants) and a `Runtime` (device, compute dtype).
It declares its tensors with `param_specs()` (local names such as "q_proj.weight"), receives
them through `load()`, and runs through `forward()`.  No part knows which model it is in.

  Norm         forward(x [T,D] float, out [T,D] activation dtype, rows=None)
  Mixer        cache_need() -> CacheNeed;  forward(h [T,H], residual [T,H] float, batch, cache)
               adds its result into `residual` (so it may fuse the sum into its last product)
  FeedForward  forward(h [T,H], residual [T,H] float, batch)       likewise adds into `residual`
  Block        forward(x [T,H] float residual stream, batch, cache) updates x in place

`h` is in the activation dtype (float32 on the 32-bit path, bfloat16 otherwise); the residual
stream is float on both paths.  `batch` is a `StepBatch`; `cache` a `CacheView`.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict

import torch

from ..cache import CacheNeed


@dataclass(frozen=True)
class ParamSpec:
    """One tensor a part needs.

    role "matrix": kept in the compute dtype (bfloat16 as stored; widened exactly on the 32-bit
    path).  role "vector": small per-channel weights, kept in float32 on both paths (a tensor
    stored in 32-bit stays so; a bfloat16 one widens exactly).  role "table": integers, int32.
    init: "normal" = N(0, 0.02); "ones_noise" = 1 + N(0, 0.1); "zeros".
    """

    shape: tuple
    role: str = "matrix"
    init: str = "normal"


class Part:
    # True if forward() takes every per-step fact (tokens, positions, lengths, pages, slots) from
    # the batch's device arrays, so that a recorded CUDA graph of a step can be replayed for later
    # steps.  A part that branches on the batch's host-side values must say False; the engine
    # then runs the model's decode steps eagerly.
    graph_safe = True

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receive device tensors, already in the dtype their role asks for."""

    def weight_bytes(self) -> int:
        """Bytes of weights one forward pass reads (for roofline arithmetic)."""
        return 0


class Norm(Part):
    def forward(self, x, out, rows=None) -> None:
        raise NotImplementedError


class Mixer(Part):
    def cache_need(self) -> CacheNeed:
        return CacheNeed()

    def forward(self, h, residual, batch, cache) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h, residual, batch) -> None:
        raise NotImplementedError


class Block(Part):
    def cache_need(self) -> CacheNeed:
        return CacheNeed()

    def forward(self, x, batch, cache) -> None:
        raise NotImplementedError
