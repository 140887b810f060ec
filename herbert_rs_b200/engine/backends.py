"""Backend names, in the manner of the reference's backend registry.

The reference keeps a static table of named backends with an availability test, an `auto`
choice and a `help` listing, and answers an unknown or unavailable name with an error that
lists what there is (crates/backend_registry/src/lib.rs:39-45, 118-189, 200-266).  This library
has two backends, both on the CUDA device: the serving precision and the true 32-bit path.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..errors import BackendError


@dataclass(frozen=True)
class BackendInfo:
    name: str
    dtype: torch.dtype
    description: str


BACKENDS = (
    BackendInfo("cuda-bf16", torch.bfloat16,
                "sm_100a kernels, bfloat16 weights/activations/cache, float accumulation (default)"),
    BackendInfo("cuda-fp32", torch.float32,
                "sm_100a kernels, everything in true float32 (no reduced-precision matrix mode)"),
)
AUTO_ORDER = ("cuda-bf16", "cuda-fp32")


def available_backends_help() -> str:
    lines = ["Available backends:"]
    for b in BACKENDS:
        lines.append(f"  {b.name:<10}  {b.description}")
    lines.append("  auto        the first of: " + ", ".join(AUTO_ORDER))
    return "\n".join(lines)


def resolve_backend(name: str = "auto") -> BackendInfo:
    if name == "auto":
        name = AUTO_ORDER[0]
    for b in BACKENDS:
        if b.name == name:
            if not torch.cuda.is_available():
                raise BackendError(f"backend '{name}' is unavailable: no CUDA device (there is no CPU backend)")
            return b
    raise BackendError(f"unknown backend '{name}'. " + available_backends_help())


def backend_for_dtype(dtype: torch.dtype) -> BackendInfo:
    for b in BACKENDS:
        if b.dtype == dtype:
            return b
    raise BackendError(f"no backend computes in {dtype}")
