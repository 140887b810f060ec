"""Random tiny configurations of the architecture against the plain implementation: head sizes
16..256 in steps of 16, 1..4 key/value heads with 1..16 query heads each, widths, vocabularies and
feed-forward widths that are no powers of two, windows on some layers, half-rotated heads, tied
and separate heads; each whole, with a decoded tail, and in batches of unequal lengths whose slots
are used again.  The seed is fixed; a failure names the configuration."""
import shutil
import tempfile

import numpy as np
import pytest

import herbert_rs_b200 as hb
import plain_qwen3 as P
from gpu_util import DTYPES, assert_close, engine_for, replay_batches, replay_tail_one_by_one, replay_whole

pytestmark = pytest.mark.gpu


def _random_config(rng):
    hd = int(rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 128, 128, 160, 256]))
    nkv = int(rng.choice([1, 2, 3, 4]))
    groups = int(rng.choice([1, 2, 3, 4, 8, 16] if hd <= 128 else [1, 2]))
    layers = int(rng.integers(1, 4))
    vocab = int(rng.choice([100, 257, 384, 1000]))
    cfg = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=vocab,
               hidden_size=int(rng.choice([48, 64, 72, 96, 136, 200, 256])), num_hidden_layers=layers,
               num_attention_heads=nkv * groups, num_key_value_heads=nkv, head_dim=hd,
               intermediate_size=int(rng.choice([56, 96, 120, 172, 256, 344])),
               rope_theta=float(rng.choice([1e4, 1e6])), rms_norm_eps=float(rng.choice([1e-6, 1e-5, 3e-6])),
               max_position_embeddings=512, tie_word_embeddings=bool(rng.integers(0, 2)), eos_token_id=vocab - 1)
    if rng.random() < 0.3:
        cfg.update(use_sliding_window=True, sliding_window=int(rng.choice([17, 40, 64, 100])),
                   layer_types=[("sliding_attention" if rng.random() < 0.6 else "full_attention") for _ in range(layers)])
    if rng.random() < 0.2 and hd >= 32:
        cfg["partial_rotary_factor"] = 0.5
    return cfg


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_configurations_in_every_cutting(seed):
    rng = np.random.default_rng(seed)
    for case in range(8):
        cfg = _random_config(rng)
        d = tempfile.mkdtemp(prefix="hb_random_")
        try:
            hb.write_random_model(cfg, d, seed=int(rng.integers(0, 1 << 30)))
            pm = P.PlainModel(d)
            reqs = [rng.integers(0, cfg["vocab_size"], int(n)).tolist()
                    for n in rng.choice([1, 2, 5, 17, 33, 64, 65, 90, 130, 200], size=4)]
            refs = [pm.logits(r).numpy() for r in reqs]
            for dtype in DTYPES:
                what = f"seed {seed} case {case} {cfg}"
                eng = engine_for(d, dtype, max_tokens=64 * 24, max_slots=4)
                i = int(rng.integers(0, 4))
                assert_close(replay_whole(eng, reqs[i]), refs[i], dtype, "whole: " + what, plain=pm, ids=reqs[i])
                assert_close(replay_tail_one_by_one(eng, reqs[i], int(rng.integers(1, 40))), refs[i], dtype, "tail: " + what, plain=pm, ids=reqs[i])
                prompt_lens = [int(rng.integers(1, len(r) + 1)) for r in reqs]
                got = replay_batches(eng, reqs, prompt_lens, [[0, 1, 2], [3]] if rng.random() < 0.5 else [[0, 1, 2, 3]])
                for g, ref, r in zip(got, refs, reqs):
                    assert_close(g, ref, dtype, "batched: " + what, plain=pm, ids=r)
                hb.ops.check_kernel_errors()
        finally:
            shutil.rmtree(d, ignore_errors=True)
