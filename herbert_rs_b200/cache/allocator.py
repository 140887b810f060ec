"""Host-side bookkeeping of reusable integer resources (sequence slots, cache pages).

The reference creates one cache per request and drops it afterwards
(crates/backends/backend_common/src/cpu_backend.rs:178-182); a batch engine hands out
slots and pages from fixed pools instead and takes them back when a batch ends.  The pool
refuses what would corrupt it: an id that is out of range, freed twice, or not held.
"""

from __future__ import annotations

import heapq
from typing import Iterable, List

from ..errors import CacheError


class IdPool:
    """A pool of the ids 0..n-1.  Lowest free id first, so reuse is immediate and predictable."""

    def __init__(self, n: int, what: str = "id"):
        if n < 0:
            raise CacheError(f"a pool of {what}s needs a size >= 0, got {n}")
        self.n = n
        self.what = what
        self._free: List[int] = list(range(n))  # a min-heap (a sorted list is one)
        self._held = bytearray(n)

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self.n - len(self._free)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i] == 1

    def alloc(self) -> int:
        if not self._free:
            raise CacheError(f"no free {self.what}: all {self.n} are held")
        i = heapq.heappop(self._free)
        self._held[i] = 1
        return i

    def alloc_many(self, count: int) -> List[int]:
        if count > len(self._free):
            raise CacheError(f"need {count} {self.what}s but only {len(self._free)} of {self.n} are free")
        return [self.alloc() for _ in range(count)]

    def free(self, i: int) -> None:
        if not (isinstance(i, int) and 0 <= i < self.n):
            raise CacheError(f"{self.what} {i!r} does not exist (pool of {self.n})")
        if not self._held[i]:
            raise CacheError(f"{self.what} {i} is not held: freed twice or never given out")
        self._held[i] = 0
        heapq.heappush(self._free, i)

    def free_many(self, ids: Iterable[int]) -> None:
        for i in ids:
            self.free(i)

    def check(self) -> None:
        """Invariant: every id is either free once or held, never both, none lost."""
        seen = bytearray(self.n)
        for i in self._free:
            if seen[i]:
                raise CacheError(f"{self.what} {i} is on the free list twice")
            if self._held[i]:
                raise CacheError(f"{self.what} {i} is both free and held")
            seen[i] = 1
        if sum(seen) + sum(self._held) != self.n:
            raise CacheError(f"{self.what}s were lost: {sum(seen)} free + {sum(self._held)} held != {self.n}")
