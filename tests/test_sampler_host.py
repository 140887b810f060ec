"""The host twin of the sampler against the reference's algorithm restated (no GPU)."""
import numpy as np
import pytest

from herbert_rs_b200.sampling import SamplingParams, host_argmax, host_sample, host_survivors, uniform_for
from plain_qwen3 import sample_distribution


def test_greedy_first_maximum_wins():
    assert host_argmax(np.array([0.5, 2.0, 2.0, -1.0], dtype=np.float32)) == 1
    assert host_sample(np.array([0.5, 2.0, 2.0], dtype=np.float32), SamplingParams(temperature=0.0), 0.99) == 1
    assert host_argmax(np.full(5, -np.inf, dtype=np.float32)) == 0


@pytest.mark.parametrize("t,k,p", [(0.8, 20, 0.9), (0.4, 40, 0.9), (1.0, 0, 1.0), (1.3, 0, 0.5), (0.7, 5, 1.0),
                                   (1.0, 1, 0.9), (1.0, 500, 0.95), (0.05, 0, 0.9), (2.0, 7, 0.01)])
def test_distribution_equals_the_reference_algorithm(t, k, p):
    rng = np.random.default_rng(3)
    logits = (rng.standard_normal(384) * 2.0).astype(np.float32)
    want = sample_distribution(logits, t, k, p)
    params = SamplingParams(t, k, p)
    keep, e = host_survivors(logits, params)
    got = e.astype(np.float64) / e.sum(dtype=np.float64)
    assert (got > 0).tolist() == (want > 0).tolist()
    assert np.abs(got - want).max() < 1e-6
    n = 20000
    counts = np.bincount([host_sample(logits, params, (i + 0.5) / n) for i in range(n)], minlength=384)
    assert np.abs(counts / n - want).max() < 2.0 / n + 1e-6


def test_top_k_edge_values():
    logits = np.arange(10, dtype=np.float32)
    for k, kept in [(0, 10), (1, 1), (10, 10), (99, 10), (3, 3)]:
        assert host_survivors(logits, SamplingParams(1.0, k, 1.0))[0].sum() == kept
    assert host_sample(logits, SamplingParams(1.0, 1, 1.0), 0.73) == 9
    assert host_sample(logits, SamplingParams(1.0, 0, 1e-6), 0.5) == 9    # a tiny nucleus is the top token
    assert host_sample(logits, SamplingParams(1e-4, 0, 1.0), 0.5) == 9    # temperature -> 0 approaches greedy


def test_uniform_stream():
    us = [uniform_for(42, s, t) for s in range(50) for t in range(50)]
    assert all(0.0 <= u < 1.0 for u in us) and len(set(us)) > 2400
    assert abs(np.mean(us) - 0.5) < 0.02
    assert uniform_for(42, 3, 9) == uniform_for(42, 3, 9) != uniform_for(43, 3, 9)
    assert all((u * (1 << 24)) == int(u * (1 << 24)) for u in us[:100])   # 24-bit, as sampler.rs:59-62
