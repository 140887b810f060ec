"""The pre-norm residual block: x += mixer(norm1(x)); x += ffn(norm2(x))
(crates/backends/backend_common/src/generic_layer.rs:1131-1328)."""

from __future__ import annotations

from .. import ops
from ..registry import build_part, register_part
from .base import Block


class PreNormBlock(Block):
    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.norm1 = build_part("norm", spec.norm1, rt=rt)
        self.mixer = build_part("mixer", spec.mixer, rt=rt)
        self.norm2 = build_part("norm", spec.norm2, rt=rt)
        self.ffn = build_part("ffn", spec.ffn, rt=rt)
        self._names = dict(spec.names)

    @property
    def graph_safe(self):
        return all(p.graph_safe for _, p in self.children())

    def children(self):
        return (("norm1", self.norm1), ("mixer", self.mixer), ("norm2", self.norm2), ("ffn", self.ffn))

    def param_specs(self):
        out = {}
        for local, part in self.children():
            for name, ps in part.param_specs().items():
                out[f"{self._names[local]}.{name}"] = ps
        return out

    def load(self, tensors):
        for local, part in self.children():
            prefix = self._names[local] + "."
            part.load({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)})

    def weight_bytes(self):
        return sum(p.weight_bytes() for _, p in self.children())

    def cache_need(self):
        return self.mixer.cache_need()

    chains_norms = True

    def first_norm(self):
        return self.norm1

    def _input(self, pending, norm, part, x):
        """What `part` reads: the pending norm itself if it can finish it, else the plain result."""
        if pending is not None and part.shares_norms:
            return pending
        h = self.rt.workspace.take(x.shape, self.rt.dtype)
        if pending is not None:
            ops.finish_norm(pending, h)
        else:
            norm.forward(x, h)
        return h

    def forward(self, x, batch, cache, normed=None, next_norm=None):
        share = ops.shared_norm_ok(x.shape[0], self.rt.dtype, x.shape[1])
        h = self._input(normed, self.norm1, self.mixer, x)
        mid = self.norm2.shareable() if share and self.mixer.shares_norms else None
        if self.mixer.shares_norms:
            pending = self.mixer.forward(h, x, batch, cache, next_norm=mid)
        else:
            pending = self.mixer.forward(h, x, batch, cache)
        h2 = self._input(pending, self.norm2, self.ffn, x)
        if self.ffn.shares_norms:
            return self.ffn.forward(h2, x, batch, next_norm=next_norm if share else None)
        self.ffn.forward(h2, x, batch)
        return None


register_part("block", "prenorm", PreNormBlock)
