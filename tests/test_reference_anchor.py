"""The plain implementation against the reference's own kernels (no GPU).

`tests/golden/reference_kernels_golden.npz` holds what the reference's x86 assembly kernels gave
on seeded inputs (made by `tests/golden/make_reference_kernels_golden.py`, which says which files
and which call order).  Here the plain implementation's functions compute the same quantities:

  * the BF16 product: y = W bf16(x), weights [out, in] row-major, the activation rounded to
    bfloat16 (nearest even) first: `linear(bf16_storage(x), W)`;
  * attention of 8 query heads over one key/value head: raw dot products, softmax weights, and
    the result of the online-softmax recurrence (m, l, o carried key by key, o / l at the end) and
    of the two-pass form: `attention_scores` (grouping of query heads, scale before the maximum,
    the maximum subtracted, weights times values).

So these formulas rest on the reference's output, not on a reading of its source alone.  What
still rests on reading: the order of the layer's steps (norm before rotation, the rotation's
pairing, which tensors a layer has), which only the reference's Rust model code shows.

The second test re-runs the reference's kernels where its sources, gcc and an AVX-512 BF16 CPU are
at hand, and checks that the stored outputs are theirs; elsewhere it is skipped.
"""
import importlib.util
import os
import shutil

import numpy as np
import pytest
import torch

import plain_qwen3 as P

HERE = os.path.dirname(os.path.abspath(__file__))
_spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_reference_kernels_golden.py"))
G = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(G)


def _t(bits):
    return torch.from_numpy(G.from_bf16_bits(bits).astype(np.float64))


def test_plain_formulas_against_the_reference_kernels_outputs():
    gold, inp = np.load(G.GOLDEN), G.inputs()
    # the product
    x = torch.from_numpy(inp["matvec_x"].astype(np.float64))
    y = P.linear(P.bf16_storage(x)[None, :], _t(inp["matvec_w"]))[0].numpy()
    assert np.abs(y - gold["matvec_y"]).max() <= 2e-5 * np.abs(y).max()
    assert np.abs(P.linear(x[None, :], _t(inp["matvec_w"]))[0].numpy() - gold["matvec_y"]).max() > 1e-3   # the rounding of x is part of it
    for i, a in enumerate(G.ATTN):
        hd, n = a["hd"], a["keys"]
        q, k, v = torch.from_numpy(inp[f"attn{i}_q"].astype(np.float64)), _t(inp[f"attn{i}_k"]), _t(inp[f"attn{i}_v"])
        scale = 1.0 / np.sqrt(hd)
        dots = (k @ q.T).numpy()                                              # [keys, heads], as the kernel lays them out
        assert np.abs(dots - gold[f"attn{i}_dots"]).max() <= 2e-5 * np.abs(dots).max()
        assert np.abs((dots * scale).max(axis=0) - gold[f"attn{i}_m"]).max() <= 1e-5
        # one query at the last of n positions, 8 query heads on 1 key/value head, through the plain function
        qq = torch.zeros(n, 8, hd, dtype=torch.float64)
        qq[-1] = q
        out = P.attention_scores(qq, k[:, None, :], v[:, None, :], scale, None)[-1].numpy()
        scale_o = np.abs(out).max()
        assert np.abs(out - gold[f"attn{i}_online"]).max() <= 1e-4 * scale_o
        assert np.abs(out - gold[f"attn{i}_twopass"]).max() <= 1e-4 * scale_o
        probs = torch.softmax(torch.from_numpy(dots * scale), dim=0).numpy()
        assert np.abs(probs - gold[f"attn{i}_probs"]).max() <= 1e-5
    # a window in the plain function hides exactly the keys it should: the same call on the kept keys alone
    w = 20
    out_w = P.attention_scores(qq, k[:, None, :], v[:, None, :], scale, w)[-1]
    out_k = P.attention_scores(qq[-w:], k[-w:, None, :], v[-w:, None, :], scale, None)[-1]
    assert torch.allclose(out_w, out_k, atol=1e-12)


def _reference_root():
    for cand in (os.environ.get("HERBERT_RS_SOURCE"), os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")):
        if cand and os.path.exists(os.path.join(cand, "crates", "backends", "backend_bf16_avx512", "src", "avx512_bf16_matvec.S")):
            return cand
    return None


def test_the_stored_outputs_are_the_reference_kernels():
    root = _reference_root()
    if root is None:
        pytest.skip("the reference's sources are not at hand")
    if shutil.which("gcc") is None:
        pytest.skip("no gcc")
    try:
        flags = open("/proc/cpuinfo").read()
    except OSError:
        flags = ""
    if "avx512_bf16" not in flags:
        pytest.skip("this CPU has no AVX-512 BF16")
    now, gold = G.run_kernels(root), np.load(G.GOLDEN)
    assert sorted(now) == sorted(gold.files)
    for name in gold.files:
        assert np.allclose(now[name], gold[name], rtol=1e-5, atol=1e-6), name     # equal bits on the CPU that made the file
