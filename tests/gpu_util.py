"""Helpers shared by the GPU tests: tolerances, replay drivers, comparison with the plain model."""
from __future__ import annotations

import numpy as np
import torch

import herbert_rs_b200 as hb

DTYPES = ["float32", "bfloat16"]

# Bounds on |engine logit - plain float64 logit|, relative to max(1, max|plain logit|).
# float32: sums of at most a few hundred float products, a handful of layers.
# bfloat16: every activation between kernels is rounded to 8 significant bits (relative 2^-9),
# and a logit is a sum over the width of such values after several layers.
TOL = {"float32": 3e-5, "bfloat16": 4e-2}


def tol_for(dtype: str, ref: np.ndarray) -> float:
    return TOL[dtype] * max(1.0, float(np.abs(ref).max()))


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
    model: four times what the number format itself does to the plain implementation (float32
    arithmetic, or bfloat16 storage between kernels), and never below the usual bound."""
    import plain_qwen3 as P
    ref = plain_model.logits(ids).numpy()
    if dtype == "float32":
        own = np.abs(plain_model.logits(ids, torch.float32).double().numpy() - ref).max()
    else:
        own = np.abs(plain_model.logits(ids, torch.float64, P.bf16_storage).numpy() - ref).max()
    return max(tol_for(dtype, ref), 4.0 * float(own))


def assert_close(got, ref, dtype, what="", bound=None):
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    err = np.abs(got - ref)
    bound = tol_for(dtype, ref) if bound is None else bound
    if not err.max() <= bound:
        row = int(np.unravel_index(np.argmax(err), err.shape)[0])
        first = int(np.argmax(err.max(axis=-1) > bound))
        raise AssertionError(f"{what} [{dtype}]: max error {err.max():.3e} > {bound:.3e}; worst row {row}, "
                             f"first row over the bound {first} of {got.shape[0]}")
    return float(err.max())
