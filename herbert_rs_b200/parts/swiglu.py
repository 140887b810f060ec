"""The dense gated feed-forward: down( silu(gate(h)) * up(h) ), added to the residual stream
(crates/backends/backend_common/src/generic_mlp.rs:83-96; silu(x) = x / (1 + exp(-x)),
kernels.rs:677-687).

gate_proj and up_proj are one matrix here.  When the intermediate size is a multiple of 8
their rows alternate in groups of 8 (8 gate rows, the 8 up rows of the same channels, ...), so
that a kernel holding 16 consecutive output columns has both halves of 8 channels; otherwise
the up rows follow all gate rows.
"""

from __future__ import annotations

import torch

from .. import ops
from ..registry import register_part
from .base import FeedForward, ParamSpec

INTERLEAVE = 8


def join_gate_up(gate: torch.Tensor, up: torch.Tensor):
    inter, hidden = gate.shape
    if inter % INTERLEAVE == 0:
        g = gate.view(inter // INTERLEAVE, INTERLEAVE, hidden)
        u = up.view(inter // INTERLEAVE, INTERLEAVE, hidden)
        return torch.cat([g, u], dim=1).reshape(2 * inter, hidden).contiguous(), INTERLEAVE
    return torch.cat([gate, up], dim=0).contiguous(), 0


class SwiGLU(FeedForward):
    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.wgu = self.wd = None
        self.interleave = 0

    def param_specs(self):
        s = self.spec
        return {
            "gate_proj.weight": ParamSpec((s.intermediate_size, s.hidden_size)),
            "up_proj.weight": ParamSpec((s.intermediate_size, s.hidden_size)),
            "down_proj.weight": ParamSpec((s.hidden_size, s.intermediate_size)),
        }

    def load(self, tensors):
        self.wgu, self.interleave = join_gate_up(tensors["gate_proj.weight"], tensors["up_proj.weight"])
        self.wd = tensors["down_proj.weight"].contiguous()

    def weight_bytes(self):
        return (self.wgu.numel() + self.wd.numel()) * self.wgu.element_size()

    shares_norms = True

    def forward(self, h, residual, batch, next_norm=None):
        ws, T, inter = self.rt.workspace, h.shape[0], self.spec.intermediate_size
        act = ws.take((T, inter), h.dtype)
        ops.gemm_swiglu(h, self.wgu, act, self.interleave, ws.take)
        return ops.gemm(act, self.wd, residual, ops.EPI_RESIDUAL, next_norm=next_norm, scratch=ws.take)


register_part("ffn", "swiglu", SwiGLU)
