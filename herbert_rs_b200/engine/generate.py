"""The generation loop: batches of unequal prompts, stop tokens, sequences that end earlier,
and as many batches one after another as there are requests.

The reference's loop serves one sequence (crates/cli/src/main.rs:1000-1009 first token from the
prompt's logits; :1241-1376 `for _ in 0..max_tokens { decode_next; sample; push; stop checks }`).
Kept from it: the stop token is part of the output (main.rs:1272, 1357); `ignore_eos`
(main.rs:94-96); the repetition detector (crates/core/src/decode_utils.rs:14-33: the same
pattern of 6..100 tokens three times in a row); the statistics' definitions (main.rs:1443-1459:
prefill tok/s = prompt tokens / prefill seconds; decode tok/s = (generated - 1) / decode seconds).

The loop only decides; it talks to the engine through three calls (`alloc_slot`, `free_slot`,
`step_and_choose`), so its decisions are tested on the CPU with a stand-in engine.
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

from ..errors import CacheError, RequestError
from ..sampling import SamplingParams, uniform_for

MIN_PATTERN, MAX_PATTERN, REPEATS = 6, 100, 3  # crates/core/src/decode_utils.rs:15-17


def detect_repetition_loop(tokens: Sequence[int]) -> Optional[int]:
    """Length of a pattern that the last tokens repeat three times, or None."""
    n = len(tokens)
    for pat in range(MIN_PATTERN, MAX_PATTERN + 1):
        need = pat * REPEATS
        if n < need:
            continue
        base = n - need
        first = tokens[base:base + pat]
        if all(tokens[base + r * pat: base + (r + 1) * pat] == first for r in range(1, REPEATS)):
            return pat
    return None


@dataclass
class GenerationOptions:
    max_tokens: int = 2048            # crates/cli/src/main.rs:90-92
    stop_token_ids: Optional[Sequence[int]] = None  # None: the model's own (config eos_token_id)
    ignore_eos: bool = False
    repeat_check: bool = False
    max_batch: Optional[int] = None   # most sequences of one batch; None: as many as there are slots
    prefill_chunk_size: Optional[int] = None  # prompts enter in pieces of at most this many tokens (crates/cli/src/main.rs:110-112)


@dataclass
class GenerationStats:
    prompt_tokens: int = 0
    generated_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0
    decode_steps: int = 0
    batches: int = 0

    @property
    def prefill_tokens_per_second(self) -> float:
        return self.prompt_tokens / self.prefill_seconds if self.prefill_seconds > 0 else 0.0

    @property
    def decode_tokens_per_second(self) -> float:
        n = self.generated_tokens - self.first_tokens
        return n / self.decode_seconds if self.decode_seconds > 0 else 0.0

    first_tokens: int = 0


@dataclass
class GenerationResult:
    tokens: List[List[int]]
    finish_reasons: List[str]
    stats: GenerationStats = field(default_factory=GenerationStats)


def plan_batches(n_requests: int, max_batch: int) -> List[List[int]]:
    """Requests in their order, cut into batches of at most max_batch."""
    if max_batch <= 0:
        raise RequestError("max_batch must be > 0")
    return [list(range(i, min(i + max_batch, n_requests))) for i in range(0, n_requests, max_batch)]


def plan_prefill_pieces(lengths: Sequence[int], chunk: Optional[int]) -> List[List[Tuple[int, int, int]]]:
    """The steps in which prompts of these lengths enter the cache when no sequence may bring more
    than `chunk` tokens to a step: a list of steps, each a list of (request, begin, end).  Every
    request's last piece lies in the last step (there its first token is chosen and all go on
    together), so a shorter prompt starts later; pieces of a request are consecutive steps."""
    if chunk is None or chunk <= 0 or max(lengths) <= chunk:
        return [[(i, 0, n) for i, n in enumerate(lengths)]]
    pieces = [-(-n // chunk) for n in lengths]
    n_steps = max(pieces)
    steps: List[List[Tuple[int, int, int]]] = [[] for _ in range(n_steps)]
    for i, n in enumerate(lengths):
        first = n_steps - pieces[i]
        # the first piece takes the remainder, so that the last one is as long as the others' last
        head = n - (pieces[i] - 1) * chunk
        begin = 0
        for j in range(pieces[i]):
            end = begin + (head if j == 0 else chunk)
            steps[first + j].append((i, begin, end))
            begin = end
    return steps


def generate(engine, prompts: Sequence[Sequence[int]], options: Optional[GenerationOptions] = None,
             sampling: Optional[SamplingParams] = None, stop_token_ids: Optional[Sequence[int]] = None
             ) -> GenerationResult:
    """Generate for every prompt; results keep the order of the requests.

    `engine` needs: alloc_slot(), free_slot(slot), step_and_choose(entries, params, uniforms) -> ids,
    step(entries, None) when prompts enter in pieces, and optionally `default_stop_token_ids`,
    `max_slots` and `admit(pairs)` (for (slot, new positions) pairs in order of priority: which of
    them fit into the next step together).  An engine that also has `launch_and_choose`, `chosen`
    and `can_continue_on_device` is kept one step ahead: the next step is queued, with its tokens
    taken on the device, before the host has read the one before; what the host does with a
    step's ids (stop checks, bookkeeping) then runs beside the GPU, not between its steps.  With `admit`, a batch takes only the prompts that fit
    (the others wait for the next batch), and a sequence that runs out of room ends alone.
    finish_reason is one of: "stop_token", "max_tokens", "repetition", "capacity".
    """
    options = options or GenerationOptions()
    sampling = sampling or SamplingParams()
    sampling.validate()
    if options.max_tokens < 0:
        raise RequestError("max_tokens must be >= 0")
    prompts = [list(p) for p in prompts]
    for i, p in enumerate(prompts):
        if not p:
            raise RequestError(f"request {i}: the prompt is empty")
    stops = stop_token_ids if stop_token_ids is not None else options.stop_token_ids
    if stops is None:
        stops = getattr(engine, "default_stop_token_ids", ())
    stops = set() if options.ignore_eos else set(int(s) for s in stops)
    seed = sampling.resolved_seed()
    max_slots = getattr(engine, "max_slots", None)
    max_batch = options.max_batch or max_slots or len(prompts) or 1
    if max_slots:
        max_batch = min(max_batch, max_slots)       # a batch larger than the engine has slots is cut, not refused

    out: List[List[int]] = [[] for _ in prompts]
    reasons: List[str] = ["max_tokens"] * len(prompts)
    stats = GenerationStats()
    if options.max_tokens == 0:
        return GenerationResult(out, reasons, stats)

    def finished(i: int, tok: int) -> Optional[str]:
        if tok in stops:
            return "stop_token"
        if len(out[i]) >= options.max_tokens:
            return "max_tokens"
        if options.repeat_check and detect_repetition_loop(out[i]) is not None:
            return "repetition"
        return None

    admit = getattr(engine, "admit", None)      # which of these (slot, new positions) fit the next step together

    def fits(pairs: List[Tuple[int, int]]) -> List[bool]:
        return list(admit(pairs)) if admit is not None else [True] * len(pairs)

    pending = list(range(len(prompts)))
    while pending:
        # the next batch: requests in their order, as many as have slots and room for their prompts
        batch_ids, slots = [], {}
        flying = None
        try:
            cand = pending[:max_batch]
            for i in cand:
                slots[i] = engine.alloc_slot()
            ok = fits([(slots[i], len(prompts[i])) for i in cand])
            if not ok[0]:
                # the first in line has the whole cache before it and still does not fit: it never will
                reasons[cand[0]] = "capacity"
                pending.remove(cand[0])
                continue
            for i, good in zip(cand, ok):
                if good:
                    batch_ids.append(i)
                else:
                    engine.free_slot(slots.pop(i))
            # a request that did not fit waits for the next batch; the ones behind it keep their order
            pending = [i for i in pending if i not in batch_ids]
            stats.batches += 1
            # all prompts in one step, or in pieces whose last ones meet in one step
            t0 = time.perf_counter()
            uni = None if sampling.greedy else [uniform_for(seed, i, 0) for i in batch_ids]     # argmax draws nothing
            steps = plan_prefill_pieces([len(prompts[i]) for i in batch_ids], options.prefill_chunk_size)
            try:
                for pieces in steps[:-1]:
                    engine.step([(slots[batch_ids[j]], prompts[batch_ids[j]][b:e]) for j, b, e in pieces], None)
                toks = engine.step_and_choose([(slots[batch_ids[j]], prompts[batch_ids[j]][b:e]) for j, b, e in steps[-1]],
                                              sampling, uni)
            except CacheError:
                # an engine without `admit`, or one whose answer did not hold: this batch ends here,
                # earlier batches keep their results and later ones still run
                for i in batch_ids:
                    reasons[i] = "capacity"
                continue
            stats.prefill_seconds += time.perf_counter() - t0
            stats.prompt_tokens += sum(len(prompts[i]) for i in batch_ids)
            active = []
            for i, tok in zip(batch_ids, toks):
                out[i].append(int(tok))
                r = finished(i, int(tok))
                if r is None:
                    active.append(i)
                else:
                    reasons[i] = r
            stats.first_tokens += len(batch_ids)
            # then one token each, for the sequences that still run
            t0 = time.perf_counter()
            ahead = all(hasattr(engine, a) for a in ("launch_and_choose", "chosen", "can_continue_on_device"))
            flying = None          # (ticket, requests) of a queued step whose ids the host has not read yet
            while active or flying is not None:
                if flying is None:
                    # only the sequences that have no room left end with "capacity" (a length limit reached,
                    # or no page left for the ones that need a new one); they give their pages back at once,
                    # and the others go on
                    ok = fits([(slots[i], 1) for i in active])
                    if not all(ok):
                        for i, good in zip(active, ok):
                            if not good:
                                reasons[i] = "capacity"
                                engine.free_slot(slots.pop(i))
                        active = [i for i, good in zip(active, ok) if good]
                        if not active:
                            break
                    uni = None if sampling.greedy else [uniform_for(seed, i, len(out[i])) for i in active]
                    entries = [(slots[i], [out[i][-1]]) for i in active]
                    try:
                        if ahead:
                            flying = (engine.launch_and_choose(entries, sampling, uni), list(active))
                        else:
                            toks = engine.step_and_choose(entries, sampling, uni)
                    except CacheError:
                        for i in active:
                            reasons[i] = "capacity"
                        break
                    stats.decode_steps += 1
                    if not ahead:
                        still = []
                        for i, tok in zip(active, toks):
                            out[i].append(int(tok))
                            r = finished(i, int(tok))
                            if r is None:
                                still.append(i)
                            else:
                                reasons[i] = r
                        active = still
                        continue
                # A step is queued.  Unless one of its sequences is sure to end with it (max_tokens) or has no
                # room for another position, the step after it is queued before its ids are read: that step
                # takes them on the device.  A sequence that turns out to have ended (a stop token, a
                # repetition) has then run one token too far; that token is dropped.
                ticket, ids = flying
                nxt = None
                if ids == active and all(len(out[i]) + 1 < options.max_tokens for i in ids) \
                        and engine.can_continue_on_device([slots[i] for i in ids]) and all(fits([(slots[i], 1) for i in ids])):
                    uni = None if sampling.greedy else [uniform_for(seed, i, len(out[i]) + 1) for i in ids]
                    try:
                        nxt = (engine.launch_and_choose([(slots[i], None) for i in ids], sampling, uni), ids)
                        stats.decode_steps += 1
                    except CacheError:
                        nxt = None
                toks = engine.chosen(ticket)
                still = []
                for i, tok in zip(ids, toks):
                    if i not in active:
                        continue                       # ended a step ago: this token is one too many
                    out[i].append(int(tok))
                    r = finished(i, int(tok))
                    if r is None:
                        still.append(i)
                    else:
                        reasons[i] = r
                        if nxt is not None and hasattr(engine, "truncate"):
                            # the queued step takes it one position too far: given back at once (a page, if it
                            # was a new one), so that the others find the room they would have found
                            try:
                                engine.truncate(slots[i], engine.length(slots[i]) - 1)
                            except CacheError:
                                pass                   # a model whose cache cannot step back keeps the position
                active = still
                flying = nxt
            stats.decode_seconds += time.perf_counter() - t0
        finally:
            if flying is not None:
                engine.chosen(flying[0])        # an error above left a queued step unread
            for s in slots.values():
                engine.free_slot(s)
        if hasattr(engine, "check_kernels"):
            engine.check_kernels()      # a kernel that gave up on a bounded wait invalidates the batch
    stats.generated_tokens = sum(len(o) for o in out)
    return GenerationResult(out, reasons, stats)
