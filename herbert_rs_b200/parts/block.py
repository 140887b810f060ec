"""The pre-norm residual block: x += mixer(norm1(x)); x += ffn(norm2(x))
(crates/backends/backend_common/src/generic_layer.rs:1131-1328)."""

from __future__ import annotations

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

    def forward(self, x, batch, cache):
        ws = self.rt.workspace
        h = ws.take(x.shape, self.rt.dtype)
        self.norm1.forward(x, h)
        self.mixer.forward(h, x, batch, cache)
        h2 = ws.take(x.shape, self.rt.dtype)
        self.norm2.forward(x, h2)
        self.ffn.forward(h2, x, batch)


register_part("block", "prenorm", PreNormBlock)
