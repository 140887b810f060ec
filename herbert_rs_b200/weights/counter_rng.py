"""Normal random numbers addressed by (key, element index): the host twin of `csrc/fill.cu`.

A tensor of a random model is `mean + std * normal(key, i)` for element i, with the key taken
from (seed, tensor name).  Values depend on nothing else: not on the device, the order in which
tensors are made, or how the elements are cut into pieces.  The device kernel and this file give
the same bits because both use only operations that round alike everywhere: 64-bit integer
mixing, exact integer-to-float conversions, and float32 add, multiply, divide and square root one
at a time (no fused multiply-add); logarithm, sine and cosine are short polynomials of those.

The reference has no random-weights mode; this exists so that tests and measurements need no
download and so that a model made on the device can also be written out and read by anyone.
"""

from __future__ import annotations

import hashlib

import numpy as np
import torch

_M64 = (1 << 64) - 1
_GOLD, _C1, _C2 = 0x9E3779B97F4A7C15, 0xBF58476D1CE4E5B9, 0x94D049BB133111EB
_CHUNK = 1 << 22


def tensor_key(seed: int, name: str) -> int:
    """64 bits from (seed, tensor name)."""
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little")


def _i64(v: int) -> int:
    v &= _M64
    return v - (1 << 64) if v >= (1 << 63) else v


def _shr(z: torch.Tensor, k: int) -> torch.Tensor:
    """Logical right shift of 64-bit patterns held in int64."""
    return (z >> k) & ((1 << (64 - k)) - 1)


def _f(bits: int) -> torch.Tensor:
    return torch.tensor(np.array(bits, dtype=np.uint32).view(np.float32).item(), dtype=torch.float32)


def _mix(key: int, idx: torch.Tensor) -> torch.Tensor:
    z = (idx + 1) * _i64(_GOLD) + _i64(key)               # int64 arithmetic wraps like uint64
    z = (z ^ _shr(z, 30)) * _i64(_C1)
    z = (z ^ _shr(z, 27)) * _i64(_C2)
    return z ^ _shr(z, 31)


def _normal_from_bits(z: torch.Tensor) -> torch.Tensor:
    f32 = torch.float32
    # radius = sqrt(-2 ln u), u = (2a + 1) / 2^24
    n = (2 * _shr(z, 41) + 1).to(torch.int32)
    nb = n.to(f32).view(torch.int32)
    e = (nb >> 23) - 127
    m = ((nb & 0x7FFFFF) | 0x3F800000).view(f32)
    big = m > _f(0x3FB504F3)
    m = torch.where(big, m * 0.5, m)
    e = e + big.to(torch.int32)
    s = (m + (-1.0)) / (m + 1.0)
    s2 = s * s
    p = s2 * _f(0x3DE38E39) + _f(0x3E124925)
    p = s2 * p + _f(0x3E4CCCCD)
    p = s2 * p + _f(0x3EAAAAAB)
    p = s2 * p + 1.0
    lnm = (s * 2.0) * p
    lnu = (e - 24).to(f32) * _f(0x3F317218) + lnm
    # numpy's square root is the hardware's, correctly rounded; torch's CPU sqrt is not (about 0.7 % of
    # float32 results are one unit off), which would break the agreement with the device kernel
    radius = torch.from_numpy(np.sqrt((lnu * -2.0).numpy()))
    # cos(2 pi t / 2^25)
    t = (_shr(z, 16) & 0x1FFFFFF).to(torch.int32)
    quadrant = t >> 23
    g = 2 * (t & 0x7FFFFF) + 1
    fold = g > 0x800000
    g = torch.where(fold, 0x1000000 - g, g)
    x = g.to(f32) * _f(0x33C90FDB)
    x2 = x * x
    sn = x2 * _f(0x3638EF1D) + _f(0xB9500D01)
    sn = x2 * sn + _f(0x3C088889)
    sn = x2 * sn + _f(0xBE2AAAAB)
    sn = (x2 * x) * sn + x
    cs = x2 * _f(0xB493F27E) + _f(0x37D00D01)
    cs = x2 * cs + _f(0xBAB60B61)
    cs = x2 * cs + _f(0x3D2AAAAB)
    cs = x2 * cs + (-0.5)
    cs = x2 * cs + 1.0
    c_in = torch.where(fold, sn, cs)
    s_in = torch.where(fold, cs, sn)
    c = torch.where(quadrant == 0, c_in, torch.where(quadrant == 1, -s_in, torch.where(quadrant == 2, -c_in, s_in)))
    return radius * c


def normal(key: int, n: int, mean: float, std: float, dtype: torch.dtype = torch.float32, start: int = 0) -> torch.Tensor:
    """Elements start .. start+n-1 of the stream `key` on the CPU, as `dtype` (float32 or bfloat16,
    rounded to nearest even)."""
    out = torch.empty(n, dtype=dtype)
    mean_t, std_t = torch.tensor(mean, dtype=torch.float32), torch.tensor(std, dtype=torch.float32)
    for lo in range(0, n, _CHUNK):
        hi = min(n, lo + _CHUNK)
        idx = torch.arange(start + lo, start + hi, dtype=torch.int64)
        v = std_t * _normal_from_bits(_mix(key, idx)) + mean_t
        out[lo:hi] = v.to(dtype)
    return out
