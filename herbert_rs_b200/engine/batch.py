"""The description of one step: which tokens of which sequences run, and where they stand.

Tokens of all sequences are packed one after another ([T] rows, no padding), so a sequence of
one token and a sequence of a thousand sit in the same matrices and nothing a padded row could
disturb exists.  Everything the kernels need is a handful of int32 arrays, built on the host,
written into one pinned buffer and copied to the device with one transfer:

  token_ids[T]   the ids                   tok_seq[T]   index of the token's sequence in this step
  positions[C,T] position in its sequence  seq_slot[B]  cache slot of each sequence
                 (C components; tok_pos = component 0)
  seq_start[B+1] first row of each sequence seq_pos0[B] cached length before this step
  seq_len[B]     length after this step    want_rows[R] rows whose logits are asked for
  pages[g][B,P]  physical page of each logical page, per key/value group
  uniforms[B]    one uniform per sequence for sampling (float bits)

The reference's step has one sequence and takes its position from the cache length
(crates/backends/backend_common/src/generic_model.rs:530; linear_ops.rs:374: start_pos + t);
the same rule gives tok_pos here, per sequence.  A model whose position encoding takes several
numbers per token (`ModelSpec.position_components`) gets as many rows; each defaults to the same
rule and can be given by the caller instead.  Component 0 is always the index in the sequence: it
is what the cache and the causal mask go by.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch


def _align(n: int, a: int = 4) -> int:
    return (n + a - 1) // a * a


@dataclass
class StepLayout:
    """Offsets (in int32 elements) of each array inside the step buffer."""

    T: int
    B: int
    R: int
    G: int
    P: int
    C: int = 1
    offsets: dict = field(default_factory=dict)
    total: int = 0

    @staticmethod
    def make(T: int, B: int, R: int, G: int, P: int, C: int = 1) -> "StepLayout":
        lay = StepLayout(T, B, R, G, P, C)
        o = 0
        for name, n in (("token_ids", T), ("tok_seq", T), ("tok_pos", C * _align(T)), ("seq_slot", B), ("seq_start", B + 1),
                        ("seq_pos0", B), ("seq_len", B), ("want_rows", max(R, 1)), ("uniforms", B)):
            lay.offsets[name] = o
            o += _align(n)
        for g in range(G):
            lay.offsets[f"pages{g}"] = o
            o += _align(B * P)
        lay.total = o
        return lay


class StepBatch:
    """Host facts and device views of one step."""

    def __init__(self, slots: Sequence[int], tokens: Sequence[Sequence[int]], pos0: Sequence[int],
                 want: Sequence[Sequence[int]], num_kv_groups: int, pages_width: Optional[int] = None,
                 page_size: int = 64, position_components: int = 1, positions: Optional[Sequence] = None):
        self.slots = list(slots)
        self.q_lens = [len(t) for t in tokens]
        self.pos0 = list(pos0)
        self.n_seqs = len(self.slots)
        self.n_tokens = sum(self.q_lens)
        self.is_decode = all(n == 1 for n in self.q_lens)
        self.max_q_len = max(self.q_lens)
        self.max_kv_len = max(p + n for p, n in zip(self.pos0, self.q_lens))
        self.page_size = page_size
        need_pages = -(-self.max_kv_len // page_size)
        self.pages_width = max(need_pages, pages_width or 0, 1)
        starts = np.zeros(self.n_seqs + 1, dtype=np.int32)
        np.cumsum(self.q_lens, out=starts[1:])
        self.seq_start_host = starts
        rows: List[int] = []
        for b, w in enumerate(want):
            for i in w:
                rows.append(int(starts[b]) + int(i))
        self.want_rows_host = rows
        self.n_want = len(rows)
        self.n_components = int(position_components)
        self.layout = StepLayout.make(self.n_tokens, self.n_seqs, self.n_want, num_kv_groups, self.pages_width,
                                      self.n_components)
        self._tokens = tokens
        self._positions = positions      # per sequence: [len, C] (or [len] when C == 1), or None
        self.host: Optional[np.ndarray] = None
        self.dev: Optional[torch.Tensor] = None
        self.pages: List[torch.Tensor] = []

    def fill_host(self, buf: np.ndarray, page_rows: Sequence[np.ndarray], uniforms: Optional[np.ndarray] = None) -> None:
        """Write every array into `buf` (int32, at least layout.total long)."""
        lay, o = self.layout, self.layout.offsets
        T, B = self.n_tokens, self.n_seqs
        flat = np.fromiter((t for seq in self._tokens for t in seq), dtype=np.int64, count=T)
        buf[o["token_ids"]:o["token_ids"] + T] = flat
        reps = np.asarray(self.q_lens, dtype=np.int64)
        seq_idx = np.repeat(np.arange(B, dtype=np.int32), reps)
        buf[o["tok_seq"]:o["tok_seq"] + T] = seq_idx
        pos0 = np.asarray(self.pos0, dtype=np.int32)
        within = np.arange(T, dtype=np.int32) - np.repeat(self.seq_start_host[:-1], reps)
        own = pos0[seq_idx] + within
        row = _align(T)
        for c in range(self.n_components):
            at = o["tok_pos"] + c * row
            buf[at:at + T] = own
            if c > 0 and self._positions is not None:
                given = np.concatenate([np.asarray(p, dtype=np.int64).reshape(len(p), -1)[:, c] for p in self._positions])
                buf[at:at + T] = given
        buf[o["seq_slot"]:o["seq_slot"] + B] = np.asarray(self.slots, dtype=np.int32)
        buf[o["seq_start"]:o["seq_start"] + B + 1] = self.seq_start_host
        buf[o["seq_pos0"]:o["seq_pos0"] + B] = pos0
        buf[o["seq_len"]:o["seq_len"] + B] = pos0 + reps.astype(np.int32)
        if self.n_want:
            buf[o["want_rows"]:o["want_rows"] + self.n_want] = np.asarray(self.want_rows_host, dtype=np.int32)
        u = np.zeros(B, dtype=np.float32) if uniforms is None else np.asarray(uniforms, dtype=np.float32)
        buf[o["uniforms"]:o["uniforms"] + B] = u.view(np.int32)
        for g, rows in enumerate(page_rows):
            buf[o[f"pages{g}"]:o[f"pages{g}"] + B * lay.P] = rows.reshape(-1)
        self.host = buf

    def bind(self, dev: torch.Tensor) -> None:
        """Create the device views over `dev` (int32, holding a copy of the host buffer)."""
        lay, o = self.layout, self.layout.offsets
        T, B = self.n_tokens, self.n_seqs
        self.dev = dev
        self.token_ids = dev[o["token_ids"]:o["token_ids"] + T]
        self.tok_seq = dev[o["tok_seq"]:o["tok_seq"] + T]
        row = _align(T)
        self.positions = dev[o["tok_pos"]:o["tok_pos"] + self.n_components * row].view(self.n_components, row)[:, :T]
        self.tok_pos = self.positions[0]
        self.seq_slot = dev[o["seq_slot"]:o["seq_slot"] + B]
        self.seq_start = dev[o["seq_start"]:o["seq_start"] + B + 1]
        self.seq_pos0 = dev[o["seq_pos0"]:o["seq_pos0"] + B]
        self.seq_len = dev[o["seq_len"]:o["seq_len"] + B]
        self.want_rows = dev[o["want_rows"]:o["want_rows"] + max(self.n_want, 1)]
        self.uniforms = dev[o["uniforms"]:o["uniforms"] + B].view(torch.float32)
        self.pages = [dev[o[f"pages{g}"]:o[f"pages{g}"] + B * lay.P].view(B, lay.P) for g in range(lay.G)]
