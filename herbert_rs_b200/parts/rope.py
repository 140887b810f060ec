"""Rotary position encoding: the cos/sin tables a mixer rotates with.

Reference (crates/backends/backend_common/src/loader_common.rs:179-202), all in float32:
  inv_freq_i = 1 / theta^(2i / rot)   for i < rot/2
  angle(pos, i) = float(pos) * inv_freq_i;  tables cos, sin of shape [max_position, rot/2].
The rotation itself pairs element j with j + rot/2 (kernels.rs:739-759) and is fused into the
mixer's cache-write kernel.
"""

from __future__ import annotations

import torch

from ..registry import register_part
from .base import Part


def rope_tables(rotary_dim: int, theta: float, max_position: int):
    """float32 tables on the CPU; every intermediate is float32, as in the reference."""
    half = rotary_dim // 2
    i = torch.arange(half, dtype=torch.float32)
    exponent = (2.0 * i) / torch.tensor(float(rotary_dim), dtype=torch.float32)
    inv_freq = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float32), exponent)
    pos = torch.arange(max_position, dtype=torch.float32)
    ang = pos[:, None] * inv_freq[None, :]
    return torch.cos(ang).contiguous(), torch.sin(ang).contiguous()


_TABLES: dict = {}


class RotaryEncoding(Part):
    """Holds the tables on the device; equal specs on one device share them."""

    def __init__(self, spec, rt):
        self.rotary_dim = spec.rotary_dim
        self.max_position = spec.max_position
        key = (spec.rotary_dim, float(spec.theta), spec.max_position, str(rt.device))
        if key not in _TABLES:
            cos, sin = rope_tables(spec.rotary_dim, spec.theta, spec.max_position)
            _TABLES[key] = (cos.to(rt.device), sin.to(rt.device))
        self.cos, self.sin = _TABLES[key]


register_part("position", "rope", RotaryEncoding)
