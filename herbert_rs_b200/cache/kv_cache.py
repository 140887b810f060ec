"""The sequence cache: paged keys/values per layer group, and fixed-size state per sequence.

What a mixer needs is declared as a `CacheNeed`; schedule steps with equal needs share a
group, and every group has storage of its own:

* key/value groups: one tensor [entries, 2, pages, kv_heads, page_size, head_dim]; a sequence
  holds a list of pages per group (logical page i = positions i*page_size ...).  A group with a
  window gives pages back as soon as no future query can reach them.
* state groups: one tensor [entries, slots, *shape], zeroed when a slot is handed out.

A slot stands for one sequence of a batch: its length, its pages, its state rows.  Slots and
pages go back to their pools when the batch ends and are used again by the next one.

The reference keeps the same things per request in `KvStore`
(crates/backends/backend_common/src/kv_cache.rs:100-129 per-layer key/value vectors,
:274-282 fixed-size state vectors that stay empty for attention-only models,
:389-406 truncate/length).  Layout here: all positions of one kv head inside a page are
contiguous, so the query heads of a group read each key tile once.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..errors import CacheError
from .allocator import IdPool


@dataclass(frozen=True)
class KVNeed:
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None  # None: all keys stay; n: only the last n are ever read


@dataclass(frozen=True)
class StateNeed:
    shape: tuple
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class CacheNeed:
    kv: Optional[KVNeed] = None
    state: Optional[StateNeed] = None


@dataclass
class CacheView:
    """What one schedule step's mixer sees of the cache."""

    kv_group: Optional[int] = None      # index into StepBatch.pages
    k: Optional[torch.Tensor] = None    # [pages, kv_heads, page_size, head_dim]
    v: Optional[torch.Tensor] = None
    writes_kv: bool = True              # False: this step reads what another step stored
    state: Optional[torch.Tensor] = None  # [slots, *shape]
    page_size: int = 0


class SequenceCache:
    def __init__(self, needs: Sequence[CacheNeed], reads_cache_of: Sequence[Optional[int]],
                 num_pages: int, num_slots: int, page_size: int = 64, max_seq_len: Optional[int] = None,
                 dtype: torch.dtype = torch.bfloat16, device=None):
        if page_size <= 0 or page_size % 16 != 0:
            raise CacheError(f"page_size must be a positive multiple of 16, got {page_size}")
        if num_pages <= 0 or num_slots <= 0:
            raise CacheError("the cache needs at least one page and one slot")
        self.page_size = page_size
        self.num_pages = num_pages
        self.num_slots = num_slots
        self.dtype = dtype
        self.device = device
        cap = num_pages * page_size
        self.max_seq_len = cap if max_seq_len is None else min(max_seq_len, cap)
        self.max_pages_per_seq = -(-self.max_seq_len // page_size)

        # group the schedule steps by need
        self.kv_needs: List[KVNeed] = []
        self.state_needs: List[StateNeed] = []
        self._kv_entries: List[List[int]] = []
        self._state_entries: List[List[int]] = []
        self.step_kv: List[Optional[tuple]] = []      # per step: (group, entry, writes)
        self.step_state: List[Optional[tuple]] = []   # per step: (group, entry)
        for i, need in enumerate(needs):
            src = reads_cache_of[i]
            if src is not None:
                if not (0 <= src < i) or reads_cache_of[src] is not None:
                    raise CacheError(f"schedule step {i} reads the cache of step {src}, which must be an earlier step that stores")
                if needs[src].kv is None or need.kv is None or \
                        (needs[src].kv.num_kv_heads, needs[src].kv.head_dim) != (need.kv.num_kv_heads, need.kv.head_dim):
                    raise CacheError(f"schedule step {i} cannot read the cache of step {src}: key/value shapes differ")
                g, e, _ = self.step_kv[src]
                self.step_kv.append((g, e, False))
            elif need.kv is not None:
                if need.kv not in self.kv_needs:
                    self.kv_needs.append(need.kv)
                    self._kv_entries.append([])
                g = self.kv_needs.index(need.kv)
                self._kv_entries[g].append(i)
                self.step_kv.append((g, len(self._kv_entries[g]) - 1, True))
            else:
                self.step_kv.append(None)
            if need.state is not None:
                if need.state not in self.state_needs:
                    self.state_needs.append(need.state)
                    self._state_entries.append([])
                g = self.state_needs.index(need.state)
                self._state_entries[g].append(i)
                self.step_state.append((g, len(self._state_entries[g]) - 1))
            else:
                self.step_state.append(None)

        self.slots = IdPool(num_slots, "slot")
        self.pools = [IdPool(num_pages, f"page of group {g}") for g in range(len(self.kv_needs))]
        self.lengths = [0] * num_slots
        self._pages: List[List[List[int]]] = [[[] for _ in self.kv_needs] for _ in range(num_slots)]
        self._released: List[List[int]] = [[0] * len(self.kv_needs) for _ in range(num_slots)]

        self.kv: List[torch.Tensor] = []
        self.state: List[torch.Tensor] = []
        if device is not None:
            for g, need in enumerate(self.kv_needs):
                self.kv.append(torch.zeros(
                    (len(self._kv_entries[g]), 2, num_pages, need.num_kv_heads, page_size, need.head_dim),
                    dtype=dtype, device=device))
            for g, need in enumerate(self.state_needs):
                self.state.append(torch.zeros((len(self._state_entries[g]), num_slots, *need.shape),
                                              dtype=need.dtype, device=device))

    # -- sizes -----------------------------------------------------------------------------
    @property
    def num_kv_groups(self) -> int:
        return len(self.kv_needs)

    def bytes_per_token(self) -> int:
        es = torch.empty((), dtype=self.dtype).element_size()
        return sum(2 * len(e) * n.num_kv_heads * n.head_dim * es for n, e in zip(self.kv_needs, self._kv_entries))

    # -- slots -----------------------------------------------------------------------------
    def alloc_slot(self) -> int:
        s = self.slots.alloc()
        self.lengths[s] = 0
        self._pages[s] = [[] for _ in self.kv_needs]
        self._released[s] = [0] * len(self.kv_needs)
        for st in self.state:
            st[:, s].zero_()
        return s

    def free_slot(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot!r} is not held: freed twice or never given out")
        for g, pages in enumerate(self._pages[slot]):
            self.pools[g].free_many(p for p in pages if p >= 0)
        self._pages[slot] = [[] for _ in self.kv_needs]
        self.lengths[slot] = 0
        self.slots.free(slot)

    def _held(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot!r} is not held")

    def length(self, slot: int) -> int:
        self._held(slot)
        return self.lengths[slot]

    # -- pages -----------------------------------------------------------------------------
    def pages_needed(self, slot: int, n_new: int) -> int:
        """Pages that `n_new` more positions of `slot` take from the fullest-used pool: the most any
        key/value group needs (groups differ once a window has given pages back)."""
        want = -(-(self.lengths[slot] + n_new) // self.page_size)
        return max((max(0, want - len(self._pages[slot][g])) for g in range(len(self.kv_needs))), default=0)

    def free_pages(self) -> int:
        """Pages free in the group with the fewest free pages."""
        return min((p.free_count for p in self.pools), default=self.num_pages)

    def reserve(self, requests: Sequence[tuple]) -> None:
        """Make room for n_new more positions per (slot, n_new); all or nothing."""
        seen = set()
        for slot, n_new in requests:
            self._held(slot)
            if slot in seen:
                raise CacheError(f"slot {slot} appears twice in one step")
            seen.add(slot)
            if n_new <= 0:
                raise CacheError("a sequence must bring at least one token")
            if self.lengths[slot] + n_new > self.max_seq_len:
                raise CacheError(
                    f"slot {slot}: {self.lengths[slot]} cached + {n_new} new positions exceed the limit of {self.max_seq_len}")
        for g in range(len(self.kv_needs)):
            need = sum(max(0, -(-(self.lengths[s] + n) // self.page_size) - len(self._pages[s][g])) for s, n in requests)
            if need > self.pools[g].free_count:
                raise CacheError(
                    f"cache full: the step needs {need} more pages of group {g}, {self.pools[g].free_count} of {self.num_pages} are free")
        for slot, n_new in requests:
            want = -(-(self.lengths[slot] + n_new) // self.page_size)
            for g in range(len(self.kv_needs)):
                pages = self._pages[slot][g]
                while len(pages) < want:
                    pages.append(self.pools[g].alloc())

    def advance(self, slot: int, n: int) -> None:
        """The step has stored n more positions; windows let go of what fell out of reach."""
        self._held(slot)
        self.lengths[slot] += n
        L = self.lengths[slot]
        for g, need in enumerate(self.kv_needs):
            if need.window is None:
                continue
            first_needed = L - need.window + 1  # the next query, at position L, reads from here
            upto = max(0, first_needed) // self.page_size
            pages = self._pages[slot][g]
            for i in range(self._released[slot][g], min(upto, len(pages))):
                if pages[i] >= 0:
                    self.pools[g].free(pages[i])
                    pages[i] = -1
            self._released[slot][g] = max(self._released[slot][g], min(upto, len(pages)))

    def truncate(self, slot: int, n: int) -> None:
        """Forget positions n.. (crates/backends/backend_common/src/kv_cache.rs:389-406)."""
        self._held(slot)
        if not (0 <= n <= self.lengths[slot]):
            raise CacheError(f"cannot truncate slot {slot} of length {self.lengths[slot]} to {n}")
        for g, need in enumerate(self.kv_needs):
            if need.window is not None and self._released[slot][g] * self.page_size > max(0, n - need.window + 1):
                raise CacheError(f"slot {slot}: positions before {n} of windowed group {g} were already given back")
        if self.state_needs and n != self.lengths[slot]:
            raise CacheError("fixed-size state cannot be rolled back: truncate is refused for this model")
        keep = -(-n // self.page_size)
        for g in range(len(self.kv_needs)):
            pages = self._pages[slot][g]
            while len(pages) > keep:
                p = pages.pop()
                if p >= 0:
                    self.pools[g].free(p)
        self.lengths[slot] = n

    def page_rows(self, group: int, slots: Sequence[int], width: int) -> np.ndarray:
        """int32 [len(slots), width]: logical page -> physical page (0 where none is held)."""
        out = np.zeros((len(slots), width), dtype=np.int32)
        for r, s in enumerate(slots):
            pages = self._pages[s][group]
            if len(pages) > width:
                raise CacheError(f"slot {s} holds {len(pages)} pages, more than the table width {width}")
            if pages:
                row = np.asarray(pages, dtype=np.int32)
                np.maximum(row, 0, out=row)
                out[r, : len(pages)] = row
        return out

    def pages_of(self, slot: int, group: int) -> List[int]:
        return list(self._pages[slot][group])

    # -- views -----------------------------------------------------------------------------
    def view(self, step: int) -> CacheView:
        v = CacheView(page_size=self.page_size)
        kv = self.step_kv[step]
        if kv is not None:
            g, e, writes = kv
            v.kv_group, v.writes_kv = g, writes
            if self.kv:
                v.k, v.v = self.kv[g][e, 0], self.kv[g][e, 1]
        st = self.step_state[step]
        if st is not None and self.state:
            g, e = st
            v.state = self.state[g][e]
        return v

    def check(self) -> None:
        """Invariants of the bookkeeping: nothing lost, nothing held twice."""
        self.slots.check()
        for g, pool in enumerate(self.pools):
            pool.check()
            owners: Dict[int, int] = {}
            for s in range(self.num_slots):
                for p in self._pages[s][g]:
                    if p < 0:
                        continue
                    if not self.slots.is_held(s):
                        raise CacheError(f"free slot {s} still lists page {p} of group {g}")
                    if p in owners:
                        raise CacheError(f"page {p} of group {g} is held by slots {owners[p]} and {s}")
                    if not pool.is_held(p):
                        raise CacheError(f"slot {s} lists page {p} of group {g}, which the pool thinks is free")
                    owners[p] = s
            if len(owners) != pool.held_count:
                raise CacheError(f"group {g}: {pool.held_count} pages are held but slots list {len(owners)}")
