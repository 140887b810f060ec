"""RMSNorm: y = (x / sqrt(mean(x^2) + eps)) * w, in float
(crates/backends/backend_common/src/kernels.rs:54-64)."""

from __future__ import annotations

from .. import ops
from ..registry import register_part
from .base import Norm, ParamSpec


class RMSNorm(Norm):
    def __init__(self, spec, rt):
        self.dim, self.eps, self.rt = spec.dim, spec.eps, rt
        self.weight = None

    def param_specs(self):
        return {"weight": ParamSpec((self.dim,), role="vector", init="ones_noise")}

    def load(self, tensors):
        self.weight = tensors["weight"].contiguous()

    def weight_bytes(self):
        return self.dim * 4

    def forward(self, x, out, rows=None):
        ops.rmsnorm(x, self.weight, out, self.eps, rows)

    def shareable(self):
        return (self.weight, self.eps)


register_part("norm", "rmsnorm", RMSNorm)
