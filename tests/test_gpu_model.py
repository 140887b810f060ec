"""The engine against the plain implementation, in every way of cutting the work."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import herbert_rs_b200 as hb
from gpu_util import (DTYPES, assert_close, bound_for, bf16_own_error, engine_for, random_ids, replay_batches, replay_tail_one_by_one,
                      replay_whole, sensitivity_bound, to_np)
from plain_qwen3 import PlainModel

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def plain(model_dirs):
    return {k: PlainModel(v) for k, v in model_dirs.items()}


@pytest.fixture(scope="module")
def sharp_dir(tmp_path_factory, model_dirs):
    """Tiny B with the q/k head-norm weights scaled up: scores spread out, so that attention looks
    at few keys and a single wrong, missing or stale key changes the logits visibly."""
    from herbert_rs_b200.weights import ModelFiles, save_file
    d = str(tmp_path_factory.mktemp("tiny_Bsharp"))
    files = ModelFiles(model_dirs["B"])
    t = {n: files.tensor(n) for n in files.names()}
    for n in t:
        if n.endswith("q_norm.weight") or n.endswith("k_norm.weight"):
            t[n] = (t[n].float() * 4.0).to(torch.bfloat16)
    save_file(t, os.path.join(d, "model.safetensors"))
    with open(os.path.join(d, "config.json"), "w") as f:
        f.write(open(os.path.join(model_dirs["B"], "config.json")).read())
    return d


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_each_request_alone_and_whole(model_dirs, plain, name, dtype):
    eng = engine_for(model_dirs[name], dtype)
    rng = np.random.default_rng(5)
    V, P = plain[name].cfg["V"], plain[name].cfg["P"]
    for n in [1, 2, 13, 64, 65, min(P, 200)] + ([300] if name == "D" else []):
        ids = random_ids(rng, V, n)
        assert_close(replay_whole(eng, ids), plain[name].logits(ids).numpy(), dtype, f"{name} whole n={n}", plain=plain[name], ids=ids)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_last_32_tokens_one_by_one(model_dirs, plain, name, dtype):
    eng = engine_for(model_dirs[name], dtype)
    rng = np.random.default_rng(6)
    for n in [33, 70, 100]:
        ids = random_ids(rng, plain[name].cfg["V"], n)
        ref = plain[name].logits(ids).numpy()
        got = replay_tail_one_by_one(eng, ids, 32)
        assert_close(got, ref, dtype, f"{name} tail n={n}", plain=plain[name], ids=ids)
        assert_close(got, replay_whole(eng, ids), dtype, f"{name} tail vs whole n={n}", plain=plain[name], ids=ids)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "Bsharp"])
def test_unequal_batches_one_after_another(model_dirs, sharp_dir, plain, name, dtype):
    d = sharp_dir if name == "Bsharp" else model_dirs[name]
    pm = PlainModel(d) if name == "Bsharp" else plain[name]
    rng = np.random.default_rng(7)
    lens = [40, 9, 75, 1, 66, 20, 5, 90, 33]
    prompts = [31, 5, 64, 1, 60, 13, 1, 70, 2]
    reqs = [random_ids(rng, pm.cfg["V"], n) for n in lens]
    # few pages (64 tokens each): the second and third batch must reuse what the first gave back
    eng = engine_for(d, dtype, max_tokens=64 * 5, max_slots=4)
    got = replay_batches(eng, reqs, prompts, [[0, 1, 2, 3], [4, 5, 6], [7, 8]])
    for i, ids in enumerate(reqs):
        bound = sensitivity_bound(pm, ids, dtype) if name == "Bsharp" else None
        assert_close(got[i], pm.logits(ids).numpy(), dtype, f"{name} batched request {i} (len {lens[i]})", bound, plain=pm, ids=ids)
    assert eng.cache.slots.free_count == 4 and all(p.free_count == 5 for p in eng.cache.pools)


@pytest.mark.parametrize("dtype", DTYPES)
def test_batch_composition_does_not_change_logits(model_dirs, plain, dtype):
    eng = engine_for(model_dirs["B"], dtype)
    rng = np.random.default_rng(8)
    reqs = [random_ids(rng, 384, n) for n in (50, 3, 17)]
    alone = [replay_whole(eng, r) for r in reqs]
    together = replay_batches(eng, reqs, [len(r) for r in reqs], [[0, 1, 2]])
    # float32: one kernel for every size, the same sums per row.  bfloat16: a step of few rows and
    # a step of many rows take different product kernels, so rounding (and only rounding) differs.
    for a, b, ids in zip(alone, together, reqs):
        assert np.abs(a - b).max() <= (1e-6 if dtype == "float32" else bound_for(plain["B"], ids, dtype, a))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C"])
def test_long_decoding(model_dirs, plain, name, dtype):
    n = {"A": 128, "C": 300}[name]           # A: up to its position limit; C: several pages, past its window
    eng = engine_for(model_dirs[name], dtype)
    ids = random_ids(np.random.default_rng(9), plain[name].cfg["V"], n)
    got = replay_tail_one_by_one(eng, ids, n - 3)
    assert_close(got, plain[name].logits(ids).numpy(), dtype, f"{name} long decode", plain=plain[name], ids=ids)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_first_tokens_of_a_sequence(model_dirs, plain, name, dtype):
    eng = engine_for(model_dirs[name], dtype)
    ids = random_ids(np.random.default_rng(10), plain[name].cfg["V"], 4)
    ref = plain[name].logits(ids).numpy()
    assert_close(replay_tail_one_by_one(eng, ids, 3), ref, dtype, f"{name} first tokens", plain=plain[name], ids=ids)
    s = eng.alloc_slot()
    first = to_np(eng.step([(s, ids[:1])], "last"))
    assert_close(first, ref[:1], dtype, "the very first token", plain=plain[name], ids=ids, rows=[0])
    assert eng.step([(s, ids[1:2])], None) is None            # nothing wanted: nothing returned
    assert_close(to_np(eng.step([(s, ids[2:4])], [[1]])), ref[3:4], dtype, "after a silent step", plain=plain[name], ids=ids, rows=[3])
    eng.free_slot(s)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompt_cut_into_pieces(model_dirs, plain, dtype):
    eng = engine_for(model_dirs["C"], dtype)
    ids = random_ids(np.random.default_rng(11), 300, 150)
    s = eng.alloc_slot()
    rows = []
    for a, b in [(0, 7), (7, 64), (64, 65), (65, 140), (140, 150)]:
        rows.append(to_np(eng.step([(s, ids[a:b])], "all")))
    eng.free_slot(s)
    assert_close(np.concatenate(rows, 0), plain["C"].logits(ids).numpy(), dtype, "prompt in pieces", plain=plain["C"], ids=ids)


@pytest.mark.parametrize("dtype", DTYPES)
def test_truncate_and_refeed(model_dirs, plain, dtype):
    eng = engine_for(model_dirs["A"], dtype)
    ids = random_ids(np.random.default_rng(12), 256, 90)
    s = eng.alloc_slot()
    eng.step([(s, ids)], None)
    eng.truncate(s, 70)
    other = ids[:70] + random_ids(np.random.default_rng(13), 256, 20)
    got = to_np(eng.step([(s, other[70:])], "all"))
    eng.free_slot(s)
    assert_close(got, plain["A"].logits(other).numpy()[70:], dtype, "after truncate", plain=plain["A"], ids=other, rows=range(70, 90))


def test_requests_are_validated_before_anything_runs(model_dirs):
    eng = engine_for(model_dirs["A"], "float32", max_tokens=128)
    s = eng.alloc_slot()
    with pytest.raises(hb.RequestError, match="outside the vocabulary"):
        eng.step([(s, [1, 256])])
    with pytest.raises(hb.RequestError, match="at least one token"):
        eng.step([(s, [])])
    with pytest.raises(hb.RequestError, match="at least one sequence"):
        eng.step([])
    with pytest.raises(hb.RequestError, match="wanted place"):
        eng.step([(s, [1, 2])], [[2]])
    with pytest.raises(hb.CacheError, match="twice in one step"):
        eng.step([(s, [1]), (s, [2])])
    with pytest.raises(hb.CacheError, match="exceed the limit of 128"):
        eng.step([(s, [1] * 129)])
    with pytest.raises(hb.CacheError, match="not held"):
        eng.step([(3, [1])])
    assert eng.length(s) == 0
    eng.free_slot(s)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_run_program(model_dirs, plain, tmp_path, dtype):
    """bin/trace_run as a user runs it: steps on standard input, logits in files."""
    rng = np.random.default_rng(14)
    a, b, c = (random_ids(rng, 256, n) for n in (40, 6, 70))
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}, {"id": "b", "tokens": b[:5], "want": [4]}], "end": []}]
    for k in range(10):
        e = [{"id": "a", "tokens": [a[30 + k]], "want": [0]}]
        if k == 0:
            e.append({"id": "b", "tokens": [b[5]], "want": [0]})
        steps.append({"step": k + 1, "entries": e, "end": ["b"] if k == 0 else (["a"] if k == 9 else [])})
    steps.append({"step": 11, "entries": [{"id": "c", "tokens": c, "want": []}], "end": []})
    steps.append({"step": 12, "entries": [{"id": "c", "tokens": [9], "want": [0]}], "end": ["c"]})
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dirs["A"], "--dtype", dtype,
                        "--out", str(out), "--max-tokens", "128", "--timing"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    ra, rb = plain["A"].logits(a).numpy(), plain["A"].logits(b).numpy()
    rc = plain["A"].logits(c + [9]).numpy()
    g0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(3, 256)
    assert_close(g0[:2].astype(np.float64), np.stack([ra[0], ra[29]]), dtype, "trace step 0", plain=plain["A"], ids=a, rows=[0, 29])
    assert_close(g0[2:].astype(np.float64), rb[4:5], dtype, "trace step 0, second request", plain=plain["A"], ids=b, rows=[4])
    g1 = np.fromfile(out / "1.f32", dtype="<f4").reshape(2, 256)
    assert_close(g1[:1].astype(np.float64), ra[30:31], dtype, "trace step 1", plain=plain["A"], ids=a, rows=[30])
    assert_close(g1[1:].astype(np.float64), rb[5:6], dtype, "trace step 1, second request", plain=plain["A"], ids=b, rows=[5])
    g10 = np.fromfile(out / "10.f32", dtype="<f4").reshape(1, 256)
    assert_close(g10.astype(np.float64), ra[39:40], dtype, "trace step 10", plain=plain["A"], ids=a, rows=[39])
    assert not (out / "11.f32").exists()
    # --timing: one line per step with its device time and, per row of the step's file, request and position
    index = [json.loads(l) for l in open(out / "index.jsonl")]
    assert [e["step"] for e in index] == [s["step"] for s in steps] and all(e["ms"] > 0 for e in index)
    assert index[0]["rows"] == [{"row": 0, "id": "a", "position": 0}, {"row": 1, "id": "a", "position": 29}, {"row": 2, "id": "b", "position": 4}]
    assert index[1]["rows"] == [{"row": 0, "id": "a", "position": 30}, {"row": 1, "id": "b", "position": 5}] and index[1]["tokens"] == 2
    assert index[11]["rows"] == [] and index[12]["rows"] == [{"row": 0, "id": "c", "position": 70}]
    g12 = np.fromfile(out / "12.f32", dtype="<f4").reshape(1, 256)
    assert_close(g12.astype(np.float64), rc[70:71], dtype, "trace step 12", plain=plain["A"], ids=c + [9], rows=[70])


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(model_dirs, plain, dtype):
    eng = engine_for(model_dirs["B"], dtype)
    rng = np.random.default_rng(15)
    prompts = [random_ids(rng, 384, n) for n in (9, 1, 30, 4, 17)]
    res = hb.generate(eng, prompts, hb.GenerationOptions(max_tokens=12, ignore_eos=True, max_batch=3),
                      hb.SamplingParams(temperature=0.0))
    assert res.stats.batches == 2 and all(len(t) == 12 for t in res.tokens)
    same = 0
    for p, got in zip(prompts, res.tokens):
        ids = list(p)
        for tok in got:
            ref = plain["B"].logits(ids)[-1].numpy()
            # the plain model's best token, or one tied with it within twice the logits' own bound
            margin = 1e-4 if dtype == "float32" else 2 * bound_for(plain["B"], ids, dtype, ref, rows=[len(ids) - 1])
            assert ref.max() - ref[tok] <= margin
            same += int(tok == int(ref.argmax()))
            ids.append(tok)
    if dtype == "float32":
        assert same == 60
    eng.cache.check()
    assert eng.cache.slots.free_count == eng.cache.num_slots


@pytest.mark.parametrize("dtype", DTYPES)
def test_generation_with_prompts_in_pieces(model_dirs, plain, dtype):
    """--prefill-chunk-size: prompts enter the cache five tokens at a time, shorter ones later, and
    the tokens are those of whole prompts (float32: identical; bfloat16: the plain model's best)."""
    eng = engine_for(model_dirs["A"], dtype)
    rng = np.random.default_rng(25)
    prompts = [random_ids(rng, 256, n) for n in (23, 2, 11, 5)]
    opt = dict(max_tokens=6, ignore_eos=True)
    whole = hb.generate(eng, prompts, hb.GenerationOptions(**opt), hb.SamplingParams(temperature=0.0))
    cut = hb.generate(eng, prompts, hb.GenerationOptions(prefill_chunk_size=5, **opt), hb.SamplingParams(temperature=0.0))
    for p, got in zip(prompts, cut.tokens):
        ids = list(p)
        for tok in got:
            ref = plain["A"].logits(ids)[-1].numpy()
            margin = 1e-4 if dtype == "float32" else 2 * bound_for(plain["A"], ids, dtype, ref, rows=[len(ids) - 1])
            assert ref.max() - ref[tok] <= margin
            ids.append(tok)
    if dtype == "float32":
        assert cut.tokens == whole.tokens
    assert cut.stats.prompt_tokens == whole.stats.prompt_tokens == 41
    eng.cache.check()
    assert eng.cache.slots.free_count == eng.cache.num_slots


def test_sampled_generation_is_reproducible_and_batch_independent(model_dirs):
    eng = engine_for(model_dirs["B"], "float32")
    rng = np.random.default_rng(16)
    prompts = [random_ids(rng, 384, n) for n in (1, 7, 16, 31)]
    sp = hb.SamplingParams(temperature=0.8, top_k=20, top_p=0.9, seed=1234)
    opt = hb.GenerationOptions(max_tokens=12, ignore_eos=True)
    a = hb.generate(eng, prompts, opt, sp).tokens
    b = hb.generate(eng, prompts, opt, sp).tokens
    assert a == b
    one = hb.generate(eng, prompts, hb.GenerationOptions(max_tokens=12, ignore_eos=True, max_batch=1), sp).tokens
    assert one == a
    c = hb.generate(eng, prompts, opt, hb.SamplingParams(temperature=0.8, top_k=20, top_p=0.9, seed=99)).tokens
    assert c != a


@pytest.mark.parametrize("dtype", DTYPES)
def test_captured_decode_steps_equal_eager_ones(model_dirs, plain, dtype):
    """Decode steps replay a captured graph; the logits must be those of the eager kernels."""
    rng = np.random.default_rng(17)
    reqs = [random_ids(rng, 300, n) for n in (150, 31, 290, 77)]
    prompts = [20, 30, 3, 70]
    eager = engine_for(model_dirs["C"], dtype, use_graphs=False)
    graphed = engine_for(model_dirs["C"], dtype, use_graphs=True)
    a = replay_batches(eager, reqs, prompts, [[0, 1, 2, 3]])
    b = replay_batches(graphed, reqs, prompts, [[0, 1, 2, 3]])
    assert eager.graph_replays == 0 and graphed.graph_replays > 200
    for x, y, ids in zip(a, b, reqs):
        assert np.abs(x - y).max() <= 1e-6          # same kernels, same arithmetic
        assert_close(y, plain["C"].logits(ids).numpy(), dtype, "graphed decode", plain=plain["C"], ids=ids)


@pytest.mark.parametrize("which,dtype", [("C", "float32"), ("D", "bfloat16")])
def test_decode_steps_that_update_the_step_buffer_in_place(model_dirs, plain, which, dtype):
    """Generation's decode steps reuse the previous step's buffer; the tokens must be those of an
    engine that builds every step anew, also across page edges, early finishers and a new batch."""
    rng = np.random.default_rng(18)
    prompts = [random_ids(rng, 300, n) for n in (60, 3, 127, 64, 20)]
    opt = hb.GenerationOptions(max_tokens=80, ignore_eos=True, max_batch=3)
    fast = engine_for(model_dirs[which], dtype)          # D in bfloat16: the fused decode attention, shared norms, graphs
    slow = engine_for(model_dirs[which], dtype, use_graphs=False)
    a = hb.generate(fast, prompts, opt, hb.SamplingParams(temperature=0.7, top_k=30, top_p=0.95, seed=5)).tokens
    b = hb.generate(slow, prompts, opt, hb.SamplingParams(temperature=0.7, top_k=30, top_p=0.95, seed=5)).tokens
    assert a == b
    assert fast.fast_decode_steps > 100 and slow.fast_decode_steps == 0
    # one sequence stops early: the next step has other sequences and must not take the short cut blindly
    stop = a[0][10]
    c = hb.generate(fast, prompts[:3], hb.GenerationOptions(max_tokens=40, stop_token_ids=[stop]), hb.SamplingParams(temperature=0.7, top_k=30, top_p=0.95, seed=5)).tokens
    d = hb.generate(slow, prompts[:3], hb.GenerationOptions(max_tokens=40, stop_token_ids=[stop]), hb.SamplingParams(temperature=0.7, top_k=30, top_p=0.95, seed=5)).tokens
    assert c == d and len(c[0]) == 11
    fast.cache.check()


@pytest.mark.parametrize("key", [0, 57])
def test_the_bfloat16_bound_sees_one_dropped_key(model_dirs, plain, key):
    """The derived bfloat16 bound is tight enough to show a fault of the cache: compared with a
    reference that is wrong on purpose (head 3 of the first layer never sees key `key`), the engine's
    logits at Tiny D are out of bounds, while against the right reference they are within."""
    import plain_qwen3 as P
    pm = plain["D"]
    ids = random_ids(np.random.default_rng(1), 1000, 200)
    eng = engine_for(model_dirs["D"], "bfloat16")
    got = replay_whole(eng, ids)
    ref = pm.logits(ids).numpy()
    bound = bound_for(pm, ids, "bfloat16", ref)
    assert np.abs(got - ref).max() <= bound
    orig, calls, head = P.attention_scores, [0], 3

    def faulty(q, k, v, scale, window):
        out = orig(q, k, v, scale, window)
        if calls[0] == 0:
            T, kh = q.shape[0], head // (q.shape[1] // k.shape[1])
            s = (q[:, head] @ k[:, kh].T) * scale
            i = torch.arange(T)
            mask = i[None, :] <= i[:, None]
            mask[:, key] = False
            mask[key, key] = True
            out[:, head] = torch.softmax(s.masked_fill(~mask, float("-inf")), -1) @ v[:, kh]
        calls[0] += 1
        return out

    P.attention_scores = faulty
    try:
        wrong = pm.logits(ids).numpy()
    finally:
        P.attention_scores = orig
    over = np.abs(got - wrong).max(axis=-1) > bound
    assert over.any() and not over[:key].any()        # rows before the dropped key cannot tell


def test_a_full_cache_ends_only_the_sequence_that_needs_the_page(model_dirs):
    """Three pages for two sequences: when no page is left, the one that needs a new page ends with
    "capacity" and gives its pages back; the other goes on and generates what it generates alone.
    A prompt that no empty cache could hold ends without a token and the next request still runs."""
    rng = np.random.default_rng(31)
    prompts = [random_ids(rng, 256, 100), random_ids(rng, 256, 10), random_ids(rng, 256, 120)]
    opt = hb.GenerationOptions(max_tokens=20, ignore_eos=True)
    sp = hb.SamplingParams(temperature=0.0)
    eng = engine_for(model_dirs["A"], "float32", max_tokens=64 * 3, max_slots=2, max_seq_len=128)
    res = hb.generate(eng, prompts, opt, sp)
    alone = hb.generate(engine_for(model_dirs["A"], "float32", max_tokens=64 * 8, max_slots=1, max_seq_len=128), prompts, opt, sp)
    # request 0: 100 + 20 positions, two pages: fits.  Request 1: a second page at position 64 is never needed.
    assert res.finish_reasons[:2] == ["max_tokens", "max_tokens"] and res.tokens[:2] == alone.tokens[:2]
    # request 2: 120 prompt tokens leave 8 positions under the limit of 128
    assert res.finish_reasons[2] == "capacity" and res.tokens[2] == alone.tokens[2][:len(res.tokens[2])] and len(res.tokens[2]) == 9
    eng.cache.check()
    assert eng.cache.slots.free_count == 2 and eng.cache.free_pages() == 3
    # pages, not the limit: two sequences of 60 tokens want a second page each after four tokens; one page is left
    eng = engine_for(model_dirs["A"], "float32", max_tokens=64 * 3, max_slots=2)
    two = [random_ids(rng, 256, 60), random_ids(rng, 256, 60)]
    res = hb.generate(eng, two, opt, sp)
    one = hb.generate(engine_for(model_dirs["A"], "float32", max_tokens=64 * 8, max_slots=1), two, opt, sp)
    assert res.finish_reasons == ["max_tokens", "capacity"]
    assert res.tokens[0] == one.tokens[0] and res.tokens[1] == one.tokens[1][:5]
    eng.cache.check()
    too_long = hb.generate(eng, [random_ids(rng, 256, 64 * 3 + 1), [5, 6]], opt, sp)
    assert too_long.finish_reasons == ["capacity", "max_tokens"] and too_long.tokens[0] == [] and len(too_long.tokens[1]) == 20


def test_a_kernel_that_gave_up_is_reported_and_the_counters_start_afresh(model_dirs, plain):
    """The failure path of the bounded waits, made on the host: a non-zero error flag and arrival
    counters left mid-count (what a kernel that gave up leaves behind).  The check raises, clears
    the flag and every counter table, and the next steps are right again.  Nothing on the GPU waits
    or faults for this."""
    from herbert_rs_b200 import ops
    eng = engine_for(model_dirs["D"], "bfloat16")
    ids = random_ids(np.random.default_rng(41), 1000, 200)
    ref = plain["D"].logits(ids).numpy()
    assert_close(replay_tail_one_by_one(eng, ids, 8), ref, "bfloat16", "before", plain=plain["D"], ids=ids)   # every counter table exists now
    dev = ops.device_key(eng.rt.device)
    tables = [ops._decode_counters[dev], ops._tcgen05_ws[dev][1], ops._stream_buffers(eng.rt.device)[1], ops._work_counters[dev]]
    for t in tables:
        t.fill_(3)
    ops._error_flag(eng.rt.device).fill_(7)
    with pytest.raises(hb.BackendError, match="gave up waiting on a barrier .code 7."):
        eng.check_kernels()
    assert int(ops._error_flag(eng.rt.device).item()) == 0 and all(int(t.abs().sum().item()) == 0 for t in tables)
    eng.check_kernels()
    assert_close(replay_tail_one_by_one(eng, ids, 8), ref, "bfloat16", "after", plain=plain["D"], ids=ids)
    assert_close(replay_whole(eng, ids), ref, "bfloat16", "after, whole", plain=plain["D"], ids=ids)


@pytest.mark.gpu
def test_decode_steps_launched_ahead_of_their_predecessor_give_the_same_bits(model_dirs, plain):
    """Programmatic dependent launch: a product fetches its first weights, and the fused attention its
    first keys of earlier steps, before the kernel before them has ended.  Inside recorded graphs
    (an option, off by default) and eagerly, the logits are the bits of the plain stream order."""
    from herbert_rs_b200 import ops
    rng = np.random.default_rng(43)
    lens = [150, 63, 257]
    reqs = [random_ids(rng, 1000, n + 24) for n in lens]

    def run(**kw):
        eng = engine_for(model_dirs["D"], "bfloat16", **kw)
        slots = [eng.alloc_slot() for _ in reqs]
        rows = [to_np(eng.step([(s, r[:n]) for s, r, n in zip(slots, reqs, lens)], "last"))]
        for t in range(24):        # the second request crosses into a new page, where its only tile holds the new key
            rows.append(to_np(eng.step([(s, [r[n + t]]) for s, r, n in zip(slots, reqs, lens)], "last")))
        return np.stack(rows)

    saved = ops.options.pdl_graph, ops.options.pdl_eager
    try:
        ops.options.pdl_graph, ops.options.pdl_eager = 0, False
        base = run()
        assert_close(base[:, 0], plain["D"].logits(reqs[0]).numpy()[lens[0] - 1:lens[0] + 24], "bfloat16", "stream order",
                     plain=plain["D"], ids=reqs[0], rows=list(range(lens[0] - 1, lens[0] + 24)))
        for mode in (1, 2):
            ops.options.pdl_graph = mode
            assert np.array_equal(run(), base), f"recorded, mode {mode}"
        ops.options.pdl_graph, ops.options.pdl_eager = 0, True
        assert np.array_equal(run(use_graphs=False), base), "eager"
    finally:
        ops.options.pdl_graph, ops.options.pdl_eager = saved
        ops.set_pdl(0)


class _OneStepAtATime:
    """The engine without the calls that let `generate` run a step ahead: the plain loop."""

    def __init__(self, engine):
        self._e = engine

    def __getattr__(self, name):
        if name in ("launch_and_choose", "chosen", "can_continue_on_device"):
            raise AttributeError(name)
        return getattr(self._e, name)


@pytest.mark.gpu
@pytest.mark.parametrize("name,dtype", [("B", "float32"), ("D", "bfloat16")])
@pytest.mark.parametrize("temperature", [0.0, 0.9])
def test_generation_one_step_ahead_gives_the_plain_loops_tokens(model_dirs, name, dtype, temperature):
    """`generate` queues a decode step before it has read the ids of the one before (those stay on
    the device).  Same tokens, same reasons, also where a stop token ends a sequence one step after
    the next step was queued, where a new page is entered, and over two batches that share slots."""
    rng = np.random.default_rng(61)
    cfg = json.load(open(os.path.join(model_dirs[name], "config.json")))
    prompts = [random_ids(rng, cfg["vocab_size"], n) for n in (60, 3, 130, 17, 64)]
    sampling = hb.SamplingParams(temperature=temperature, top_k=20, seed=9)
    free_run = hb.GenerationOptions(max_tokens=40, ignore_eos=True, max_batch=3)
    eng = engine_for(model_dirs[name], dtype, max_tokens=4096)
    probe = hb.generate(_OneStepAtATime(eng), prompts, free_run, sampling)
    # stop tokens taken from what the model really emits, so that sequences end early and unforeseen
    stops = sorted({probe.tokens[0][7], probe.tokens[2][20], probe.tokens[4][1]})
    opt = hb.GenerationOptions(max_tokens=40, stop_token_ids=stops, max_batch=3)
    plain_run = hb.generate(_OneStepAtATime(eng), prompts, opt, sampling)
    before = eng.fast_decode_steps
    ahead_run = hb.generate(eng, prompts, opt, sampling)
    assert ahead_run.tokens == plain_run.tokens and ahead_run.finish_reasons == plain_run.finish_reasons
    assert "stop_token" in plain_run.finish_reasons and eng.fast_decode_steps > before
    assert not eng._open
    assert hb.generate(eng, prompts, free_run, sampling).tokens == probe.tokens
    eng.cache.check()
    assert eng.cache.slots.free_count == eng.cache.num_slots
