"""Choosing the next token: greedy, or temperature / top-k / top-p sampling.

Options and their meaning are the reference's (crates/core/src/sampler.rs:4-11, 72-145;
defaults from crates/cli/src/main.rs:130-140):
  temperature  logits are divided by it; 0 = greedy argmax, the first maximum wins   (0.4)
  top_k        keep the k largest scaled logits; 0 = off                               (40)
  top_p        after softmax over the survivors keep the shortest prefix, in descending
               probability, whose cumulative probability reaches p; 1.0 = off          (0.9)
then one uniform r in [0,1) picks the first survivor whose cumulative probability exceeds r.

Two deliberate differences, both stated in the device kernel as well: survivors are found by
value thresholds, so values exactly equal to a threshold all survive (the reference's partial
sort keeps an arbitrary one of equal values); and the cumulative draw runs in index order (the
reference draws in its sort order).  The distribution is the same.

Randomness: the reference owns one xorshift64 stream seeded by the clock (sampler.rs:21-34,
50-62).  Here every (seed, sequence, step) has its own value, so what a sequence samples does not
depend on which other sequences share its batch.  `host_sample` is the plain twin of the kernel.
"""

from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Optional

import numpy as np

_M64 = (1 << 64) - 1


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.4
    top_k: int = 40
    top_p: float = 0.9
    seed: Optional[int] = None  # None: seeded from the clock, like the reference

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0

    def validate(self) -> None:
        from ..errors import RequestError
        if self.temperature < 0.0:
            raise RequestError("temperature must be >= 0")
        if self.top_k < 0:
            raise RequestError("top_k must be >= 0")
        if not (0.0 < self.top_p <= 1.0):
            raise RequestError("top_p must be in (0, 1]")

    def resolved_seed(self) -> int:
        return self.seed if self.seed is not None else time.time_ns() & _M64


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _M64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M64
    return x ^ (x >> 31)


def uniform_for(seed: int, sequence: int, step: int) -> float:
    """A uniform float in [0,1) with 24 bits, as sampler.rs:50-62 makes them, from a state that
    depends only on (seed, sequence, step)."""
    x = _splitmix64(_splitmix64(_splitmix64(seed & _M64) ^ (sequence & _M64)) ^ (step & _M64))
    if x == 0:
        x = 0xDEADBEEF  # xorshift must not start at 0 (sampler.rs:31-33)
    x ^= (x << 13) & _M64
    x ^= x >> 7
    x ^= (x << 17) & _M64
    return float(np.float32((x >> 40) / float(1 << 24)))


def host_argmax(logits: np.ndarray) -> int:
    """First maximum wins; 0 if nothing exceeds -inf (sampler.rs:244-254)."""
    v = np.asarray(logits, dtype=np.float32)
    if v.size == 0:
        return 0
    w = np.where(np.isnan(v), -np.inf, v)
    m = w.max()
    return 0 if m == -np.inf else int(np.argmax(w == m))


def host_survivors(logits: np.ndarray, p: SamplingParams):
    """(mask of survivors, unnormalised softmax weights e_i) under the library's conventions."""
    s = (np.asarray(logits, dtype=np.float32) / np.float32(p.temperature)).astype(np.float32)
    n = s.size
    keep = np.ones(n, dtype=bool)
    if 0 < p.top_k < n:
        kth = np.sort(s)[n - p.top_k]
        keep = s >= kth
    e = np.where(keep, np.exp((s - s.max()).astype(np.float32)), np.float32(0)).astype(np.float32)
    if p.top_p < 1.0:
        total = e.sum(dtype=np.float32)
        order = np.argsort(-s, kind="stable")
        order = order[keep[order]]
        csum = np.cumsum(e[order], dtype=np.float32)
        idx = int(np.searchsorted(csum, np.float32(p.top_p) * total, side="left"))
        idx = min(idx, len(order) - 1)
        thresh = s[order[idx]]
        keep = keep & (s >= thresh)
        e = np.where(keep, e, np.float32(0)).astype(np.float32)
    return keep, e


def host_sample(logits: np.ndarray, p: SamplingParams, u: float) -> int:
    if p.greedy:
        return host_argmax(logits)
    keep, e = host_survivors(logits, p)
    csum = np.cumsum(e, dtype=np.float32)
    target = np.float32(u) * csum[-1]
    idx = int(np.searchsorted(csum, target, side="right"))
    if idx >= len(e):
        idx = int(np.nonzero(keep)[0][-1])
    return idx


def device_choose(logits, p: SamplingParams, uniforms, out) -> None:
    """tokens out[r] for logits [R, V] on the device (argmax, or the sampling kernel)."""
    from .. import ops
    if p.greedy:
        ops.argmax(logits, out)
    else:
        ops.sample(logits, p.temperature, p.top_k, p.top_p, uniforms, out)
