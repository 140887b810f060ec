"""Helpers shared by the GPU tests: tolerances, replay drivers, comparison with the plain model."""
from __future__ import annotations

import numpy as np
import torch

import herbert_rs_b200 as hb

DTYPES = ["float32", "bfloat16"]

# Bounds on |engine logit - plain float64 logit|.
# float32: relative to max(1, max|plain logit|): sums of at most a few thousand float products.
# bfloat16: derived per model and request from what the number format itself does: the plain
# implementation run in float64 with every activation that an engine keeps between two kernels
# rounded to bfloat16 (`bf16_storage`) differs from the exact plain logits by `own`; the engine may
# differ by BF16_K times that.  Measured on a B200 over all model-level comparisons of this suite
# the engine's error is 0.5 to 1.9 times `own` (the engine also rounds the softmax weights and
# uses exp2/rsqrt approximations; the maximum over a few hundred logits fluctuates), so K = 3.
# Where no plain model is at hand (a part alone, a toy model) the bound is BF16_REL times the
# largest reference value: 8 significant bits are 2^-9 relative per rounding, a few roundings deep.
TOL = {"float32": 3e-5}
BF16_K = 3.0
BF16_REL = 1.0e-2
RECORDS: list = []        # (what, error, bound, own or scale) of every bfloat16 comparison, for the session summary
_own_cache: dict = {}


def tol_for(dtype: str, ref: np.ndarray) -> float:
    if dtype == "float32":
        return TOL[dtype] * max(1.0, float(np.abs(ref).max()))
    return BF16_REL * float(np.abs(ref).max())


def bf16_own_error(plain_model, ids, rows=None, arith=torch.float64) -> float:
    """What bfloat16 storage between kernels does to the plain implementation's logits of `ids`
    (`arith`: the plain side's arithmetic; float32 where float64 would take too long: its own
    rounding is a thousand times below bfloat16's)."""
    import plain_qwen3 as P
    key = (id(plain_model), tuple(ids), None if rows is None else tuple(rows), arith)
    if key not in _own_cache:
        ref = plain_model.logits(ids, arith)
        low = plain_model.logits(ids, arith, P.bf16_storage)
        d = (low - ref).abs()
        _own_cache[key] = float((d if rows is None else d[list(rows)]).max())
    return _own_cache[key]


def bound_for(plain_model, ids, dtype: str, ref: np.ndarray, rows=None, arith=torch.float64) -> float:
    if dtype == "float32":
        return tol_for(dtype, ref)
    return BF16_K * bf16_own_error(plain_model, ids, rows, arith)


def engine_for(model_dir: str, dtype: str, max_tokens: int = 2048, **kw) -> hb.Engine:
    return hb.Engine.from_folder(model_dir, dtype=dtype, max_tokens=max_tokens, **kw)


def to_np(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy().astype(np.float64)


def replay_whole(engine, ids):
    s = engine.alloc_slot()
    out = to_np(engine.step([(s, ids)], "all"))
    engine.free_slot(s)
    return out


def replay_tail_one_by_one(engine, ids, tail=32):
    tail = min(tail, len(ids) - 1)
    s = engine.alloc_slot()
    head = len(ids) - tail
    rows = [to_np(engine.step([(s, ids[:head])], "all"))]
    for t in ids[head:]:
        rows.append(to_np(engine.step([(s, [t])], "all")))
    engine.free_slot(s)
    return np.concatenate(rows, 0)


def replay_batches(engine, requests, prompt_lens, batches):
    """requests: list of token lists; prompt_lens[i] tokens go in the first step of request i's
    batch, the rest one per step; a request that has no tokens left ends (its slot is freed at
    once).  `batches` lists request indices per batch; batches run one after another on the same
    engine.  Returns per request the logits at all of its positions."""
    got = {i: [] for i in range(len(requests))}
    for members in batches:
        slots = {i: engine.alloc_slot() for i in members}
        fed = {i: prompt_lens[i] for i in members}
        logits = to_np(engine.step([(slots[i], requests[i][:fed[i]]) for i in members], "all"))
        o = 0
        for i in members:
            got[i].append(logits[o:o + fed[i]]); o += fed[i]
        live = list(members)
        while True:
            for i in [i for i in live if fed[i] >= len(requests[i])]:
                engine.free_slot(slots.pop(i)); live.remove(i)
            if not live:
                break
            logits = to_np(engine.step([(slots[i], [requests[i][fed[i]]]) for i in live], "all"))
            for r, i in enumerate(live):
                got[i].append(logits[r:r + 1]); fed[i] += 1
        engine.cache.check()
    return [np.concatenate(got[i], 0) for i in range(len(requests))]


def random_ids(rng, vocab, n):
    return rng.integers(0, vocab, n).tolist()


def sensitivity_bound(plain_model, ids, dtype: str) -> float:
    """For a model made ill-conditioned on purpose (sharp attention), the bound follows from the
    model in float32 too: four times what float32 arithmetic does to the plain implementation,
    never below the usual bound.  bfloat16: the usual derived bound."""
    ref = plain_model.logits(ids).numpy()
    if dtype == "float32":
        own = np.abs(plain_model.logits(ids, torch.float32).double().numpy() - ref).max()
        return max(tol_for(dtype, ref), 4.0 * float(own))
    return bound_for(plain_model, ids, dtype, ref)


def assert_close(got, ref, dtype, what="", bound=None, plain=None, ids=None, rows=None, arith=torch.float64):
    """|got - ref| <= bound everywhere.  With `plain` and `ids` (and `rows`, when `ref` holds only
    those positions) the bfloat16 bound is derived from the model (see the top of this file)."""
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    err = np.abs(got - ref)
    if bound is None:
        bound = bound_for(plain, ids, dtype, ref, rows, arith) if plain is not None else tol_for(dtype, ref)
    if dtype == "bfloat16":
        RECORDS.append((what, float(err.max()), float(bound), "model" if plain is not None else "scale"))
    if not err.max() <= bound:
        row = int(np.unravel_index(np.argmax(err), err.shape)[0])
        first = int(np.argmax(err.max(axis=-1) > bound))
        raise AssertionError(f"{what} [{dtype}]: max error {err.max():.3e} > {bound:.3e}; worst row {row}, "
                             f"first row over the bound {first} of {got.shape[0]}")
    return float(err.max())
