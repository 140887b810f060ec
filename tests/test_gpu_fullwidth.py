"""One layer at Qwen3-8B widths (hidden 4096, 32/8 heads of 128, feed-forward 12288): the kernels at
the tile counts and strides they serve in production, against the plain implementation."""
import numpy as np
import pytest
import torch

import herbert_rs_b200 as hb
from gpu_util import assert_close, engine_for, random_ids, replay_batches, replay_tail_one_by_one, replay_whole
from plain_qwen3 import PlainModel

pytestmark = pytest.mark.gpu

WIDE = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=20040, hidden_size=4096,
            num_hidden_layers=1, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
            intermediate_size=12288, rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=4096,
            tie_word_embeddings=False, eos_token_id=3)


@pytest.fixture(scope="module")
def wide(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("wide"))
    hb.write_random_model(WIDE, d, seed=55)
    return d, PlainModel(d)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_cutting_at_production_widths(wide, dtype):
    d, plain = wide
    rng = np.random.default_rng(3)
    reqs = [random_ids(rng, 20040, n) for n in (150, 9, 70)]
    refs = [plain.logits(r, torch.float32).double().numpy() for r in reqs]     # float32 plain: float64 at this width is slow
    eng = engine_for(d, dtype, max_tokens=1024, max_slots=4)
    for r, ref in zip(reqs, refs):
        assert_close(replay_whole(eng, r), ref, dtype, "wide whole", plain=plain, ids=r, arith=torch.float32)
    assert_close(replay_tail_one_by_one(eng, reqs[0], 32), refs[0], dtype, "wide one by one", plain=plain, ids=reqs[0], arith=torch.float32)
    got = replay_batches(eng, reqs, [100, 9, 3], [[0, 1, 2]])
    for g, ref, r in zip(got, refs, reqs):
        assert_close(g, ref, dtype, "wide batched", plain=plain, ids=r, arith=torch.float32)
    from herbert_rs_b200 import ops
    ops.check_kernel_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_decode_batch_of_forty_at_production_widths(wide, dtype):
    """Between 17 and 64 sequences the decode step's large products go through the tensor-memory
    kernel (tiles of 128 weight rows, shared norms), the small one through the mma.sync kernel:
    forty unequal prompts in one step, then one token each, against the plain implementation."""
    d, plain = wide
    rng = np.random.default_rng(4)
    lens = [int(n) for n in rng.integers(1, 14, 40)]
    reqs = [random_ids(rng, 20040, n + 5) for n in lens]
    eng = engine_for(d, dtype, max_tokens=48 * 64, max_slots=48)
    got = replay_batches(eng, reqs, lens, [list(range(40))])
    for i in (0, 7, 19, 39):
        ref = plain.logits(reqs[i], torch.float32).double().numpy()
        assert_close(got[i], ref, dtype, f"request {i} of forty", plain=plain, ids=reqs[i], arith=torch.float32)
    from herbert_rs_b200 import ops
    ops.check_kernel_errors()
