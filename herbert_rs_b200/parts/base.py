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

Optional: a norm shared between two products.  Between "add into the residual stream" and "the
next product" lies only a norm, and for a few rows its kernel is all latency.  A mixer or
feed-forward that says `shares_norms = True` (1) accepts an `ops.PendingNorm` in place of `h` and
(2) takes a keyword `next_norm=(weight, eps)`: it may then return the PendingNorm of the residual
stream it has just updated (or None, and the caller runs the norm).  A norm offers itself for
this with `shareable()`.  Parts without the flag never see either; the block finishes or runs
the norm for them.
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
    # True if forward() accepts an ops.PendingNorm as its input and a `next_norm` keyword.
    shares_norms = False

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

    def shareable(self):
        """(weight [D] float, eps) if this is y = x * w / sqrt(mean(x^2) + eps), which a product
        before it and a product after it can compute between them; else None."""
        return None


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

    # True if forward() takes the keywords `normed` and `next_norm` below; a block without the flag is
    # called as forward(x, batch, cache) and its neighbours run their norms themselves.
    chains_norms = False

    def first_norm(self):
        """The norm this block applies to the stream before anything else, which the block before
        it may begin; None if there is none to share."""
        return None

    def forward(self, x, batch, cache, normed=None, next_norm=None):
        """Update x.  With `chains_norms`: `normed` is the PendingNorm of x under `first_norm()`,
        begun by the block before (or None); `next_norm` is the following block's first norm as
        (weight, eps); the block may return the PendingNorm of its result under it, or None."""
        raise NotImplementedError
