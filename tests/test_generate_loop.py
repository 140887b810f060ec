"""The generation loop's decisions, with a stand-in engine (no GPU)."""
import pytest

import herbert_rs_b200 as hb
from herbert_rs_b200.engine.generate import detect_repetition_loop, generate, plan_batches, plan_prefill_pieces
from herbert_rs_b200.errors import CacheError, RequestError


class FakeEngine:
    """Next token = (last token + 1) % 100; records every step; has `max_slots` slots."""

    def __init__(self, max_slots=4, capacity=None, pool=None, admits=True):
        self.pool, self.admits = pool, admits
        self.max_slots = max_slots
        self.free = list(range(max_slots))
        self.steps = []
        self.default_stop_token_ids = (50,)
        self.lengths = {}
        self.capacity = capacity
        self.uniforms = []

    def alloc_slot(self):
        s = self.free.pop(0)
        self.lengths[s] = 0
        return s

    def free_slot(self, s):
        assert s not in self.free
        self.free.append(s)
        self.free.sort()
        self.lengths[s] = 0

    def admit(self, pairs):
        """Per sequence a limit of `capacity` positions; all sequences together at most `pool` positions."""
        used = sum(self.lengths[s] for s in range(self.max_slots) if s not in self.free)
        out = []
        for s, n in pairs:
            good = (self.capacity is None or self.lengths[s] + n <= self.capacity) and \
                   (self.pool is None or used + n <= self.pool)
            if good:
                used += n
            out.append(good)
        return out if self.admits else [True] * len(pairs)

    def step(self, entries, want):
        assert want is None
        for s, t in entries:
            self.lengths[s] += len(t)
        self.steps.append([(s, list(t)) for s, t in entries])

    def step_and_choose(self, entries, params, uniforms):
        for s, t in entries:
            if self.capacity is not None and self.lengths[s] + len(t) > self.capacity:
                raise CacheError("cache full")
        for s, t in entries:
            self.lengths[s] += len(t)
        self.steps.append([(s, list(t)) for s, t in entries])
        self.uniforms.append(None if uniforms is None else list(uniforms))      # None: greedy, nothing is drawn
        return [(t[-1] + 1) % 100 for _, t in entries]


def test_unequal_prompts_then_one_token_each():
    e = FakeEngine()
    r = generate(e, [[1, 2, 3], [10], [20, 21]], hb.GenerationOptions(max_tokens=3), hb.SamplingParams(temperature=0.0))
    assert r.tokens == [[4, 5, 6], [11, 12, 13], [22, 23, 24]]
    assert r.finish_reasons == ["max_tokens"] * 3
    assert e.steps[0] == [(0, [1, 2, 3]), (1, [10]), (2, [20, 21])]      # all prompts in one step
    assert e.steps[1] == [(0, [4]), (1, [11]), (2, [22])]                # then one token each
    assert len(e.steps) == 3 and e.free == [0, 1, 2, 3]
    assert e.uniforms == [None] * 3                                      # greedy draws nothing
    assert r.stats.prompt_tokens == 6 and r.stats.generated_tokens == 9 and r.stats.decode_steps == 2


def test_stop_token_ends_a_sequence_early_and_is_kept():
    e = FakeEngine()
    r = generate(e, [[48], [10], [49]], hb.GenerationOptions(max_tokens=5), hb.SamplingParams(temperature=0.0))
    assert r.tokens[0] == [49, 50] and r.finish_reasons[0] == "stop_token"     # the stop token is part of the output
    assert r.tokens[2] == [50] and r.finish_reasons[2] == "stop_token"         # stops on its very first token
    assert r.tokens[1] == [11, 12, 13, 14, 15]
    assert e.steps[1] == [(0, [49]), (1, [11])]        # the one that ended is not stepped again
    assert e.steps[2] == [(1, [12])]                   # the batch shrinks; order is kept


def test_ignore_eos_and_user_stop_ids():
    r = generate(FakeEngine(), [[48]], hb.GenerationOptions(max_tokens=4, ignore_eos=True), hb.SamplingParams(temperature=0.0))
    assert r.tokens == [[49, 50, 51, 52]]
    r = generate(FakeEngine(), [[48]], hb.GenerationOptions(max_tokens=9, stop_token_ids=[52, 60]), hb.SamplingParams(temperature=0.0))
    assert r.tokens == [[49, 50, 51, 52]] and r.finish_reasons == ["stop_token"]


def test_more_requests_than_slots_run_as_batches_one_after_another():
    e = FakeEngine(max_slots=2)
    prompts = [[i] for i in range(5)]
    r = generate(e, prompts, hb.GenerationOptions(max_tokens=2), hb.SamplingParams(temperature=0.0))
    assert r.tokens == [[i + 1, i + 2] for i in range(5)]
    assert r.stats.batches == 3
    assert [len(s) for s in e.steps] == [2, 2, 2, 2, 1, 1]
    assert e.steps[2][0][0] == 0 and e.steps[4][0][0] == 0     # slots are used again
    assert plan_batches(5, 2) == [[0, 1], [2, 3], [4]]


def test_slots_are_freed_when_a_step_fails():
    class Broken(FakeEngine):
        def step_and_choose(self, entries, params, uniforms):
            raise RuntimeError("boom")
    e = Broken()
    with pytest.raises(RuntimeError):
        generate(e, [[1], [2]], hb.GenerationOptions(max_tokens=2), hb.SamplingParams(temperature=0.0))
    assert e.free == [0, 1, 2, 3]


def test_running_out_of_cache_ends_with_capacity():
    e = FakeEngine(capacity=4)
    r = generate(e, [[1, 2]], hb.GenerationOptions(max_tokens=10), hb.SamplingParams(temperature=0.0))
    assert r.finish_reasons == ["capacity"] and r.tokens == [[3, 4, 5]]


def test_only_the_sequence_that_runs_out_of_room_ends_with_capacity():
    # a limit of 8 positions per sequence: the long prompt reaches it after two tokens, the short one goes on
    e = FakeEngine(capacity=8)
    r = generate(e, [[1, 2, 3, 4, 5, 6], [10]], hb.GenerationOptions(max_tokens=5), hb.SamplingParams(temperature=0.0))
    assert r.finish_reasons == ["capacity", "max_tokens"]
    assert r.tokens == [[7, 8, 9], [11, 12, 13, 14, 15]]
    assert e.steps[3] == [(1, [13])]                 # the step after the long one left: the short one alone
    assert e.free == [0, 1, 2, 3]
    # the same without `admit`: the engine's error ends the whole batch (what an outside engine gets)
    e = FakeEngine(capacity=8, admits=False)
    r = generate(e, [[1, 2, 3, 4, 5, 6], [10]], hb.GenerationOptions(max_tokens=5), hb.SamplingParams(temperature=0.0))
    assert r.finish_reasons == ["capacity", "capacity"] and e.free == [0, 1, 2, 3]


def test_prompts_that_do_not_fit_together_wait_for_the_next_batch():
    # 10 positions in all: prompts of 6 and 5 cannot start together; a prompt of 12 never fits
    e = FakeEngine(pool=10)
    r = generate(e, [[1, 2, 3, 4, 5, 6], [20, 21, 22, 23, 24], list(range(30, 42)), [50]],
                 hb.GenerationOptions(max_tokens=2, ignore_eos=True), hb.SamplingParams(temperature=0.0))
    assert r.tokens == [[7, 8], [25, 26], [], [51, 52]]
    assert r.finish_reasons == ["max_tokens", "max_tokens", "capacity", "max_tokens"]
    assert e.steps[0] == [(0, [1, 2, 3, 4, 5, 6]), (3, [50])]      # who fits goes along; order of results is the requests'
    assert r.stats.batches == 2 and e.free == [0, 1, 2, 3]


def test_a_prompt_step_that_overflows_keeps_the_earlier_batches():
    class Tight(FakeEngine):
        def step_and_choose(self, entries, params, uniforms):
            if any(len(t) > 3 for _, t in entries):
                raise CacheError("cache full")
            return super().step_and_choose(entries, params, uniforms)
    e = Tight(max_slots=1, admits=False)
    r = generate(e, [[1, 2], [1, 2, 3, 4], [9]], hb.GenerationOptions(max_tokens=2), hb.SamplingParams(temperature=0.0))
    assert r.tokens == [[3, 4], [], [10, 11]] and r.finish_reasons == ["max_tokens", "capacity", "max_tokens"]
    assert e.free == [0]


def test_uniforms_depend_on_request_and_step_not_on_batch():
    a, b = FakeEngine(max_slots=4), FakeEngine(max_slots=1)
    p = hb.SamplingParams(temperature=0.8, seed=123)
    generate(a, [[1], [2], [3]], hb.GenerationOptions(max_tokens=3), p)
    generate(b, [[1], [2], [3]], hb.GenerationOptions(max_tokens=3), p)
    together = {(i, s): a.uniforms[s][i] for s in range(3) for i in range(3)}
    alone = {(i, s): b.uniforms[i * 3 + s][0] for i in range(3) for s in range(3)}
    assert together == alone
    assert len(set(together.values())) == 9 and all(0.0 <= u < 1.0 for u in together.values())


def test_bad_requests():
    with pytest.raises(RequestError, match="empty"):
        generate(FakeEngine(), [[1], []])
    with pytest.raises(RequestError, match="temperature"):
        generate(FakeEngine(), [[1]], sampling=hb.SamplingParams(temperature=-1.0))
    with pytest.raises(RequestError, match="top_p"):
        generate(FakeEngine(), [[1]], sampling=hb.SamplingParams(top_p=0.0))
    assert generate(FakeEngine(), [[1]], hb.GenerationOptions(max_tokens=0)).tokens == [[]]


def test_repetition_detector():
    # the reference's constants: patterns of 6..100 tokens, three times (decode_utils.rs:14-33)
    pat = [1, 2, 3, 4, 5, 6]
    assert detect_repetition_loop([9] + pat * 3) == 6
    assert detect_repetition_loop(pat * 2 + pat[:5]) is None
    assert detect_repetition_loop([1, 2, 3, 4, 5] * 6) == 10     # a 5-pattern shows up as a 10-pattern
    assert detect_repetition_loop([7] * 17) is None and detect_repetition_loop([7] * 18) == 6

    class Looping(FakeEngine):
        def step_and_choose(self, entries, params, uniforms):
            return [7 for _ in entries]
    r = generate(Looping(), [[1]], hb.GenerationOptions(max_tokens=100, repeat_check=True), hb.SamplingParams(temperature=0.0))
    assert r.finish_reasons == ["repetition"] and len(r.tokens[0]) == 18


@pytest.mark.parametrize("lengths,chunk", [([9, 1, 30, 4, 17], 5), ([10, 10], 5), ([3, 2], 8), ([33], 32), ([7, 64, 1], 1)])
def test_prompts_in_pieces_meet_in_the_last_step(lengths, chunk):
    steps = plan_prefill_pieces(lengths, chunk)
    assert sorted(i for i, _, _ in steps[-1]) == list(range(len(lengths)))      # everyone's last piece
    seen = {i: 0 for i in range(len(lengths))}
    active_since = {}
    for j, pieces in enumerate(steps):
        assert len({i for i, _, _ in pieces}) == len(pieces)                     # a request once per step
        for i, b, e in pieces:
            assert b == seen[i] and 0 < e - b <= max(chunk, 1) and e <= lengths[i]   # in order, no gap, no piece too long
            seen[i] = e
            active_since.setdefault(i, j)
        for i, first in active_since.items():
            assert any(k == i for k, _, _ in pieces)                             # once begun, in every step to the end
    assert seen == {i: n for i, n in enumerate(lengths)}
    assert len(steps) == max(-(-n // chunk) for n in lengths)


def test_generation_with_a_prefill_chunk_size_steps_the_pieces_then_decodes():
    e = FakeEngine()
    r = generate(e, [[1, 2, 3, 4, 5, 6, 7], [10], [20, 21, 22]],
                 hb.GenerationOptions(max_tokens=2, prefill_chunk_size=3), hb.SamplingParams(temperature=0.0))
    assert e.steps[0] == [(0, [1])]                                  # the remainder first
    assert e.steps[1] == [(0, [2, 3, 4])]
    assert e.steps[2] == [(0, [5, 6, 7]), (1, [10]), (2, [20, 21, 22])]
    assert e.steps[3] == [(0, [8]), (1, [11]), (2, [23])]
    assert r.tokens == [[8, 9], [11, 12], [23, 24]] and r.stats.prompt_tokens == 11
    whole = generate(FakeEngine(), [[1, 2, 3, 4, 5, 6, 7], [10], [20, 21, 22]],
                     hb.GenerationOptions(max_tokens=2), hb.SamplingParams(temperature=0.0))
    assert whole.tokens == r.tokens


class AheadEngine(FakeEngine):
    """The stand-in with the calls that let the loop queue a step before it has read the one before:
    tokens a step chose stay "on the device" (`last`), and a step of (slot, None) entries takes them."""

    def __init__(self, *a, stop_after=None, **kw):
        super().__init__(*a, **kw)
        self.open, self.tickets, self.last, self.from_device, self.unread_peak, self.truncated = {}, 0, None, 0, 0, 0

    def launch_and_choose(self, entries, params, uniforms):
        assert len(self.open) < 2
        if entries[0][1] is None:
            assert self.last is not None and [s for s, _ in entries] == [s for s, _ in self.last]
            entries = [(s, [t]) for (s, _), (_, t) in zip(entries, self.last)]
            self.from_device += 1
        toks = FakeEngine.step_and_choose(self, entries, params, uniforms)
        self.last = [(s, t) for (s, _), t in zip(entries, toks)]
        self.open[self.tickets] = toks
        self.unread_peak = max(self.unread_peak, len(self.open))
        self.tickets += 1
        return self.tickets - 1

    def chosen(self, ticket):
        return self.open.pop(ticket)

    def length(self, slot):
        return self.lengths[slot]

    def truncate(self, slot, n):
        assert 0 <= n <= self.lengths[slot]
        self.truncated += self.lengths[slot] - n
        self.lengths[slot] = n

    def can_continue_on_device(self, slots):
        return self.last is not None and list(slots) == [s for s, _ in self.last] and len(self.open) < 2

    def step_and_choose(self, entries, params, uniforms):
        self.last = None          # the prompts' step: its ids are read at once
        return FakeEngine.step_and_choose(self, entries, params, uniforms)


@pytest.mark.parametrize("stops,max_tokens", [((), 7), ((30,), 40), ((13, 30), 40), ((), 1), ((), 2)])
def test_a_loop_one_step_ahead_decides_as_the_plain_one(stops, max_tokens):
    prompts = [[1, 2, 3], [10], [20, 21], [27]]
    opt = hb.GenerationOptions(max_tokens=max_tokens, stop_token_ids=list(stops))
    plain, ahead = FakeEngine(), AheadEngine()
    a = generate(plain, prompts, opt, hb.SamplingParams(temperature=0.0))
    b = generate(ahead, prompts, opt, hb.SamplingParams(temperature=0.0))
    assert a.tokens == b.tokens and a.finish_reasons == b.finish_reasons
    assert not ahead.open and sorted(ahead.free) == sorted(plain.free)
    if max_tokens > 3:
        assert ahead.from_device > 0 and ahead.unread_peak == 2            # it did run ahead
    if not stops:
        assert len(ahead.steps) == len(plain.steps)                          # an end by max_tokens is foreseen: no step too many
        assert ahead.truncated == 0
    else:
        assert len(plain.steps) <= len(ahead.steps) <= len(plain.steps) + len(stops)   # one dropped token per unforeseen end
        assert ahead.truncated > 0                                                      # ... whose position is given back


def test_a_loop_one_step_ahead_draws_the_same_uniforms():
    p = hb.SamplingParams(temperature=0.8, seed=5)
    plain, ahead = FakeEngine(), AheadEngine()
    generate(plain, [[1], [2], [3]], hb.GenerationOptions(max_tokens=6), p)
    generate(ahead, [[1], [2], [3]], hb.GenerationOptions(max_tokens=6), p)
    assert plain.uniforms == ahead.uniforms


@pytest.mark.parametrize("kw", [dict(capacity=8), dict(capacity=4), dict(pool=14), dict(capacity=8, admits=False)])
def test_a_loop_one_step_ahead_runs_out_of_room_as_the_plain_one(kw):
    prompts = [[1, 2, 3, 4, 5], [10], [20, 21]]
    opt = hb.GenerationOptions(max_tokens=12, stop_token_ids=[])
    plain, ahead = FakeEngine(**kw), AheadEngine(**kw)
    a = generate(plain, prompts, opt, hb.SamplingParams(temperature=0.0))
    b = generate(ahead, prompts, opt, hb.SamplingParams(temperature=0.0))
    assert a.tokens == b.tokens and a.finish_reasons == b.finish_reasons and "capacity" in a.finish_reasons
    assert not ahead.open and ahead.free == plain.free


def test_a_batch_size_beyond_the_engines_slots_is_cut_to_them():
    e = FakeEngine(max_slots=2)
    r = generate(e, [[1], [10], [20], [30], [40]], hb.GenerationOptions(max_tokens=2, max_batch=4), hb.SamplingParams(temperature=0.0))
    assert r.tokens == [[2, 3], [11, 12], [21, 22], [31, 32], [41, 42]] and r.stats.batches == 3 and e.free == [0, 1]


@pytest.mark.parametrize("pool", range(4, 18))
def test_a_sequence_that_ends_a_step_late_leaves_the_others_the_room_it_would_have(pool):
    """One sequence ends by a stop token while the step after is already queued with it in; the
    position that step gave it is handed back, so the others run out of room exactly where they
    would have with the plain loop."""
    prompts = [[27], [1], [60, 61]]
    opt = hb.GenerationOptions(max_tokens=9, stop_token_ids=[30])
    plain, ahead = FakeEngine(pool=pool), AheadEngine(pool=pool)
    a = generate(plain, prompts, opt, hb.SamplingParams(temperature=0.0))
    b = generate(ahead, prompts, opt, hb.SamplingParams(temperature=0.0))
    assert a.tokens == b.tokens and a.finish_reasons == b.finish_reasons
    assert not ahead.open and ahead.free == plain.free
