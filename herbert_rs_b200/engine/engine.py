"""The engine: a model, its cache, and the one step function.

`step(entries, want)` runs exactly the tokens it is given, as one packed batch, from the cache
that earlier steps left, and returns float logits at the wanted places.  Sequences that start
together bring their whole prompts in one step (unequal lengths, no padding) and then one token
each; a sequence may also bring a few tokens at a time (a prompt cut into pieces).  The
reference's counterparts serve one sequence: `prefill`, `decode_next`, `continue_prefill`
(crates/core/src/backend.rs:137-158) and logits at every new position (`verify_draft_tokens`,
crates/backends/backend_common/src/generic_model.rs:737-834).

Everything is validated on the host before anything is launched, as the reference does
(generic_model.rs:140-152, 165-172, 531-537): empty input, token id >= vocab, context overflow,
and here also slot validity, room in the cache, and a slot named twice.
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ..cache import SequenceCache
from ..errors import BackendError, RequestError
from ..sampling import SamplingParams, device_choose
from .batch import StepBatch
from .runtime import Runtime, Workspace

Want = Union[str, Sequence[Sequence[int]], None]


class Engine:
    def __init__(self, model, max_tokens: int, max_slots: Optional[int] = None,
                 max_seq_len: Optional[int] = None, use_graphs: bool = True):
        if not torch.cuda.is_available() or model.rt.device.type != "cuda":
            raise BackendError("the engine runs on a CUDA device only: there is no CPU path")
        self.model = model
        self.rt: Runtime = model.rt
        ps = self.rt.page_size
        num_pages = max(1, -(-int(max_tokens) // ps))
        num_slots = max_slots if max_slots is not None else min(num_pages, 1024)
        limit = model.spec.max_position if max_seq_len is None else min(max_seq_len, model.spec.max_position)
        self.cache = SequenceCache(model.cache_needs(), model.reads_cache_of(), num_pages, num_slots,
                                   page_size=ps, max_seq_len=limit, dtype=self.rt.dtype, device=self.rt.device)
        self._host = torch.empty(1 << 14, dtype=torch.int32).pin_memory()
        self._dev = torch.empty(1 << 14, dtype=torch.int32, device=self.rt.device)
        self._tok_out = torch.empty(max(num_slots, 1), dtype=torch.int32, device=self.rt.device)
        self._copied = torch.cuda.Event()
        self._copied.record()
        # Decode steps (one token per sequence) are launch-bound: each shape of such a step is
        # captured once as a CUDA graph and replayed; lengths, pages and tokens are read from the
        # step buffer on the device, so one graph serves every later step of that shape.
        self.use_graphs = use_graphs and model.graph_safe
        self._graphs: dict = {}
        self._graph_ws = Workspace(self.rt.device)
        self._eager_ws = self.rt.workspace
        self.graph_replays = 0
        self._decode_again = None      # (slots, batch, lengths after it): lets the next decode step of the same sequences update the step buffer in place
        self._host_owner = None        # the batch whose arrays the pinned buffer holds
        self.fast_decode_steps = 0
        self.kernels_per_graph: dict = {}   # batch size -> kernels in its captured decode step
        self._chosen_on_device = False   # the step before left its chosen ids in _tok_out
        self._tok_ring = [(torch.empty(max(num_slots, 1), dtype=torch.int32).pin_memory(), torch.cuda.Event()) for _ in range(2)]
        self._tickets = 0
        self._open: dict = {}
        self.launches_last = 0
        self.h2d_bytes_last = 0
        self.d2h_bytes_last = 0

    # -- construction ------------------------------------------------------------------------
    @classmethod
    def from_folder(cls, model_dir: str, dtype: Union[str, torch.dtype] = "bfloat16", max_tokens: int = 4096,
                    max_slots: Optional[int] = None, max_seq_len: Optional[int] = None, device="cuda",
                    page_size: Optional[int] = None, use_graphs: bool = True,
                    round_weights_to_bf16: bool = False) -> "Engine":
        """An engine over the model folder.  `max_tokens` sizes the cache: the most positions that
        live sequences hold at any time, each sequence's count rounded up to whole pages
        (`pages_for`).  `round_weights_to_bf16` rounds every float tensor to bfloat16 while loading,
        norm weights included, as the reference does with a checkpoint stored in 32-bit."""
        from ..weights import load_model
        model = load_model(model_dir, device=device, dtype=_dtype(dtype), page_size=page_size,
                           round_weights_to_bf16=round_weights_to_bf16)
        return cls(model, max_tokens, max_slots, max_seq_len, use_graphs)

    @staticmethod
    def default_page_size() -> int:
        from .runtime import DEFAULT_PAGE_SIZE
        return DEFAULT_PAGE_SIZE

    @classmethod
    def pages_for(cls, tokens_per_sequence: int, sequences: int = 1, page_size: Optional[int] = None) -> int:
        """Cache pages that `sequences` sequences of `tokens_per_sequence` positions hold."""
        ps = page_size or cls.default_page_size()
        return -(-int(tokens_per_sequence) // ps) * int(sequences)

    @property
    def page_size(self) -> int:
        return self.rt.page_size

    @property
    def vocab_size(self) -> int:
        return self.model.spec.vocab_size

    @property
    def default_stop_token_ids(self) -> tuple:
        return tuple(self.model.spec.stop_token_ids)

    @property
    def max_slots(self) -> int:
        return self.cache.num_slots

    # -- slots -------------------------------------------------------------------------------
    def alloc_slot(self) -> int:
        return self.cache.alloc_slot()

    def free_slot(self, slot: int) -> None:
        self.cache.free_slot(slot)

    def check_kernels(self) -> None:
        """Raise if a kernel gave up on one of its bounded waits since the last check (reads one
        int from the device, so it waits for the work queued so far)."""
        from .. import ops
        ops.check_kernel_errors()

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    def admit(self, pairs: Sequence[Tuple[int, int]]) -> List[bool]:
        """For (slot, new positions) in order of priority: which of them fit into the next step
        together.  One does not fit if it would pass the length limit, or if the pages it needs are
        no longer free after the ones before it took theirs.  Nothing is reserved."""
        free = self.cache.free_pages()
        lengths, limit = self.cache.lengths, self.cache.max_seq_len
        if free >= len(pairs) and all(n == 1 and lengths[s] < limit for s, n in pairs):
            return [True] * len(pairs)          # one position each takes at most one page each
        out = []
        for slot, n in pairs:
            need = self.cache.pages_needed(slot, n)
            good = self.cache.length(slot) + n <= self.cache.max_seq_len and need <= free
            if good:
                free -= need
            out.append(good)
        return out

    def truncate(self, slot: int, n: int) -> None:
        self.cache.truncate(slot, n)

    # -- the step ----------------------------------------------------------------------------
    def _prepare(self, entries: Sequence[Tuple[int, Sequence[int]]], want: Want,
                 uniforms: Optional[np.ndarray] = None, pages_width: Optional[int] = None,
                 positions: Optional[Sequence] = None) -> StepBatch:
        if len(entries) == 0:
            raise RequestError("a step needs at least one sequence")
        slots = [int(s) for s, _ in entries]
        tokens = [list(t) for _, t in entries]
        V = self.vocab_size
        for s, t in zip(slots, tokens):
            if len(t) == 0:
                raise RequestError(f"slot {s}: a sequence must bring at least one token")
            bad = [x for x in t if not (isinstance(x, (int, np.integer)) and 0 <= x < V)]
            if bad:
                raise RequestError(f"slot {s}: token id {bad[0]!r} is outside the vocabulary of {V}")
        if want is None or want == "none":
            want_l: List[List[int]] = [[] for _ in tokens]
        elif want == "last":
            want_l = [[len(t) - 1] for t in tokens]
        elif want == "all":
            want_l = [list(range(len(t))) for t in tokens]
        else:
            want_l = [list(w) for w in want]
            if len(want_l) != len(tokens):
                raise RequestError("want must list places for every sequence of the step")
            for w, t in zip(want_l, tokens):
                if any(not (0 <= i < len(t)) for i in w):
                    raise RequestError(f"a wanted place is outside the {len(t)} tokens its sequence brings")
        C = self.model.spec.position_components
        if positions is not None:
            if len(positions) != len(tokens):
                raise RequestError("positions must be given for every sequence of the step")
            for p, t in zip(positions, tokens):
                shape = np.asarray(p).shape
                if shape not in ((len(t), C),) and not (C == 1 and shape == (len(t),)):
                    raise RequestError(f"positions of a sequence of {len(t)} tokens must have shape [{len(t)}, {C}], got {list(shape)}")
        self.cache.reserve([(s, len(t)) for s, t in zip(slots, tokens)])
        pos0 = [self.cache.lengths[s] for s in slots]
        if pages_width is None and self.use_graphs and all(len(t) == 1 for t in tokens):
            # a few widths only, so that a captured decode step is reused while sequences grow
            need = -(-(max(pos0) + 1) // self.rt.page_size)
            pages_width = min(max(4, 1 << (need - 1).bit_length()), max(self.cache.max_pages_per_seq, need))
        batch = StepBatch(slots, tokens, pos0, want_l, self.cache.num_kv_groups, pages_width, self.rt.page_size,
                          C, positions)
        n = batch.layout.total
        if n > self._host.numel():
            size = 1 << (n - 1).bit_length()
            self._host = torch.empty(size, dtype=torch.int32).pin_memory()
            self._dev = torch.empty(size, dtype=torch.int32, device=self.rt.device)
            self._graphs.clear()       # captured steps point into the old buffer
        rows = [self.cache.page_rows(g, slots, batch.pages_width) for g in range(self.cache.num_kv_groups)]
        self._copied.synchronize()  # the previous step's transfer has read the pinned buffer
        batch.fill_host(self._host.numpy(), rows, uniforms)
        self._dev[:n].copy_(self._host[:n], non_blocking=True)
        self._copied.record()
        self.h2d_bytes_last = n * 4
        batch.bind(self._dev)
        self._host_owner = batch
        return batch

    def _prepare_decode_again(self, entries, uniforms: Optional[np.ndarray]) -> Optional[StepBatch]:
        """The next one-token step of the sequences of the previous step: instead of building the
        step buffer anew, bump positions and lengths in place, write the new tokens (and page rows,
        when a sequence enters a new page) and upload.  None if this is not such a step.
        Entries whose tokens are None take the tokens that the previous step chose, which are
        still on the device: nothing of that step has to be known on the host."""
        st = self._decode_again
        if st is None or self._host_owner is not st[1] or st[1]._positions is not None:
            return None
        slots, batch, lens_after = st
        if len(entries) != len(slots):
            return None
        lengths = self.cache.lengths
        from_device = entries[0][1] is None
        for i, (s, t) in enumerate(entries):
            if s != slots[i] or (t is None) != from_device or (t is not None and len(t) != 1) or lengths[s] != lens_after[i] \
                    or not self.cache.slots.is_held(s):
                return None
        if from_device and not self._chosen_on_device:
            return None
        ps = self.rt.page_size
        if -(-(max(lens_after) + 1) // ps) > batch.pages_width:
            return None
        V = self.vocab_size
        toks = None if from_device else [t[0] for _, t in entries]
        if toks is not None:
            for s, x in zip(slots, toks):
                if not (isinstance(x, (int, np.integer)) and 0 <= x < V):
                    raise RequestError(f"slot {s}: token id {x!r} is outside the vocabulary of {V}")
        new_page = any(n % ps == 0 for n in lens_after)
        self.cache.reserve([(s, 1) for s in slots])
        B, o, host = len(slots), batch.layout.offsets, self._host.numpy()
        self._copied.synchronize()
        if toks is not None:
            host[o["token_ids"]:o["token_ids"] + B] = toks
        for name in ("seq_pos0", "seq_len"):
            host[o[name]:o[name] + B] += 1
        row = (B + 3) // 4 * 4
        for c in range(batch.n_components):
            host[o["tok_pos"] + c * row:o["tok_pos"] + c * row + B] += 1
        if uniforms is not None:
            host[o["uniforms"]:o["uniforms"] + B] = np.asarray(uniforms, dtype=np.float32).view(np.int32)
        if new_page:
            for g in range(self.cache.num_kv_groups):
                rows = self.cache.page_rows(g, list(slots), batch.pages_width)
                host[o[f"pages{g}"]:o[f"pages{g}"] + B * batch.pages_width] = rows.reshape(-1)
        n = batch.layout.total
        first = o["tok_seq"] if from_device else 0          # the ids are the buffer's first array
        self._dev[first:n].copy_(self._host[first:n], non_blocking=True)
        self._copied.record()
        if from_device:
            self._dev[o["token_ids"]:o["token_ids"] + B].copy_(self._tok_out[:B], non_blocking=True)
        self.h2d_bytes_last = (n - first) * 4
        self.fast_decode_steps += 1
        return batch

    def _forward(self, batch: StepBatch):
        """Logits of the step: eagerly, or by replaying the captured graph of this step's shape."""
        from .. import ops as _ops
        if not (self.use_graphs and batch.is_decode):
            self.rt.workspace = self._eager_ws
            _ops.set_pdl(1 if _ops.options.pdl_eager else 0)
            return self.model.forward(batch, self.cache)
        _ops.set_pdl(int(_ops.options.pdl_graph))
        key = (batch.n_seqs, batch.n_want, batch.pages_width)
        hit = self._graphs.get(key)
        if hit is not None:
            graph, logits = hit
            graph.replay()
            self.graph_replays += 1
            return logits
        self.rt.workspace = self._graph_ws
        try:
            self._graph_ws.frozen = False
            logits = self.model.forward(batch, self.cache)      # the real step; also sizes the arena
            self._graph_ws.rewind()                             # grows the arena if the step overflowed it
            if self._graph_ws._overflow_seen:
                self._graphs.clear()                            # older graphs point into the old arena
                self._graph_ws._overflow_seen = False
            self._graph_ws.frozen = True
            if len(self._graphs) >= 64:
                self._graphs.pop(next(iter(self._graphs)))
            graph = torch.cuda.CUDAGraph()
            before = _ops.launch_count()
            with torch.cuda.graph(graph):                       # records only; nothing runs
                captured = self.model.forward(batch, self.cache)
            self.kernels_per_graph[batch.n_seqs] = _ops.launch_count() - before
            self._graphs[key] = (graph, captured)
            return logits                                       # keeps its own storage alive
        finally:
            self._graph_ws.frozen = False
            self.rt.workspace = self._eager_ws

    def _finish(self, batch: StepBatch) -> None:
        for s, n in zip(batch.slots, batch.q_lens):
            self.cache.advance(s, n)

    def step(self, entries: Sequence[Tuple[int, Sequence[int]]], want: Want = "last",
             positions: Optional[Sequence] = None) -> Optional[torch.Tensor]:
        """Run the given tokens; return logits [wanted, vocab] (float32, on the device), in the order
        of the entries and of their wanted places.  The tensor is the engine's own buffer: it is
        overwritten by the next step, so copy what must last.

        `positions` (only for models whose `position_components` exceeds 1): per sequence an integer
        array [tokens, components]; component 0 is ignored (it is always the index in the sequence),
        the others replace the default, which is that index again."""
        batch = self._prepare(entries, want, positions=positions)
        logits = self._forward(batch)
        self._finish(batch)
        self._chosen_on_device = False
        return logits

    def step_and_choose(self, entries: Sequence[Tuple[int, Sequence[int]]], params: SamplingParams,
                        uniforms: Optional[Sequence[float]] = None) -> List[int]:
        """One step with the logits at each sequence's last token, then one token id per sequence
        chosen on the device; only the ids travel back to the host."""
        return self.chosen(self.launch_and_choose(entries, params, uniforms))

    def launch_and_choose(self, entries: Sequence[Tuple[int, Optional[Sequence[int]]]], params: SamplingParams,
                          uniforms: Optional[Sequence[float]] = None) -> int:
        """`step_and_choose` without the wait: the step is queued and a ticket for its token ids
        returned (`chosen`).  Entries (slot, None), for all sequences or none, continue the step
        before with the ids it chose, taken on the device: the host may queue a step before it has
        read the one before (`can_continue_on_device` says whether).  At most two tickets are open."""
        B = len(entries)
        if len(self._open) >= 2:
            raise RequestError("two queued steps are still unread: read one (`chosen`) before queueing another")
        u = None if uniforms is None else np.asarray(uniforms, dtype=np.float32)
        from_device = B > 0 and entries[0][1] is None
        batch = self._prepare_decode_again(entries, u) if self.use_graphs else None
        if batch is None:
            if from_device:
                raise RequestError("a step can take its tokens from the device only right after a step of the same sequences that chose them")
            batch = self._prepare(entries, "last", u)
        logits = self._forward(batch)
        self._finish(batch)
        if self.use_graphs and batch.is_decode:
            self._decode_again = (tuple(batch.slots), batch, [self.cache.lengths[s] for s in batch.slots])
        out = self._tok_out[:B]
        device_choose(logits, params, batch.uniforms, out)
        self._chosen_on_device = True
        ticket = self._tickets
        self._tickets += 1
        host, event = self._tok_ring[ticket % 2]
        host[:B].copy_(out, non_blocking=True)
        event.record()
        self._open[ticket] = B
        self.d2h_bytes_last = B * 4
        return ticket

    def chosen(self, ticket: int) -> List[int]:
        """The token ids of a queued step (waits for it)."""
        B = self._open.pop(ticket)
        host, event = self._tok_ring[ticket % 2]
        event.synchronize()
        return host[:B].tolist()

    def can_continue_on_device(self, slots: Sequence[int]) -> bool:
        """Whether `launch_and_choose([(slot, None), ...])` can follow now: the step before was a
        recorded one-token-or-prompt step of exactly these sequences whose ids were chosen on the device."""
        st = self._decode_again
        return bool(self.use_graphs and st is not None and self._chosen_on_device and self._host_owner is st[1]
                    and tuple(slots) == st[0] and len(self._open) < 2 and st[1]._positions is None
                    and all(self.cache.lengths[s] == n for s, n in zip(st[0], st[2]))
                    and -(-(max(st[2]) + 1) // self.rt.page_size) <= st[1].pages_width)


def _dtype(d) -> torch.dtype:
    if isinstance(d, torch.dtype):
        return d
    table = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
             "f32": torch.float32}
    if d not in table:
        raise BackendError(f"unknown dtype {d!r}: bfloat16 or float32")
    return table[d]
