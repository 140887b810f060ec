"""Load-time kernels: the counter-based random fill against its host twin (equal bytes), casts,
the rounding option of the loader, and a random model made on the device against its folder."""
import json
import os

import numpy as np
import pytest
import torch

import herbert_rs_b200 as hb
from herbert_rs_b200 import ops
from herbert_rs_b200.weights import ModelFiles, counter_rng, save_file
from plain_qwen3 import PlainModel
from tiny_configs import TINY

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,mean,std", [(1, 0.0, 1.0), (1000003, 0.0, 0.02), (5 * (1 << 20) + 7, 1.0, 0.1)])
def test_random_fill_gives_the_host_twins_bytes(dtype, n, mean, std):
    key = counter_rng.tensor_key(7, f"some.tensor.{n}")
    out = torch.empty(n, dtype=dtype, device="cuda")
    ops.rng_normal(out, key, mean, std)
    twin = counter_rng.normal(key, n, mean, std, dtype)
    assert torch.equal(out.cpu().view(torch.int16 if dtype == torch.bfloat16 else torch.int32),
                       twin.view(torch.int16 if dtype == torch.bfloat16 else torch.int32))
    if n > 1000:
        z = (out.double() - mean) / std
        assert abs(z.mean().item()) < 0.01 and abs(z.std().item() - 1) < 0.01 and 2.9 < (z ** 4).mean().item() < 3.1


def test_a_model_made_on_the_device_is_the_model_its_folder_holds(tmp_path):
    d = str(tmp_path / "m")
    hb.write_random_model(TINY["B"], d, seed=5)                 # numbers made on the CPU
    d2 = str(tmp_path / "m2")
    hb.write_random_model(TINY["B"], d2, seed=5, device="cuda")  # the same, made by the kernel
    assert open(os.path.join(d, "model.safetensors"), "rb").read() == open(os.path.join(d2, "model.safetensors"), "rb").read()
    rt = hb.Runtime("cuda", torch.bfloat16)
    direct = hb.Engine(hb.random_model(TINY["B"], 5, rt), max_tokens=256)
    loaded = hb.Engine.from_folder(d, dtype="bfloat16", max_tokens=256)
    ids = [5, 17, 3, 250, 9, 100, 42]
    a, b = direct.alloc_slot(), loaded.alloc_slot()
    assert torch.equal(direct.step([(a, ids)], "all"), loaded.step([(b, ids)], "all"))


@pytest.mark.parametrize("src", [torch.float32, torch.bfloat16, torch.float16])
def test_casts(src):
    torch.manual_seed(0)
    x = (torch.randn(100003) * 3).to(src)
    x[:2] = torch.tensor([1.0 + 2 ** -8, 1.0 + 3 * 2 ** -8]).to(src)      # ties of the bfloat16 rounding (exact in float32 only)
    dx = x.cuda()
    for dst in (torch.float32, torch.bfloat16):
        got = ops.cast(dx, dst)
        assert got.dtype == dst and torch.equal(got.cpu(), x.to(dst))
        if src == dst:
            assert got is dx
    r = ops.cast(dx, torch.float32, round_bf16=True)
    assert torch.equal(r.cpu(), x.float().to(torch.bfloat16).float())
    f = torch.empty(1001, dtype=torch.bfloat16, device="cuda")
    ops.fill(f, 1.5)
    assert (f == 1.5).all()
    i = torch.empty(77, dtype=torch.int32, device="cuda")
    ops.fill(i, 9)
    assert (i == 9).all()


def test_round_weights_to_bf16_on_a_folder_stored_in_32_bit(tmp_path):
    """A checkpoint stored in F32 whose values are not bfloat16 values: without the option the 32-bit
    path computes with the stored values; with it every float tensor, norm weights included, is
    rounded first, which is the reference's arithmetic.  The plain implementation on a folder that
    holds the rounded values is the reference for the second."""
    src = str(tmp_path / "bf")
    hb.write_random_model(TINY["A"], src, seed=3)
    files = ModelFiles(src)
    g = torch.Generator().manual_seed(1)
    exact = {n: files.tensor(n).float() * (1 + 2e-3 * torch.randn(files.tensor(n).shape, generator=g)) for n in files.names()}
    files.close()
    f32_dir, rounded_dir = str(tmp_path / "f32"), str(tmp_path / "rounded")
    for d, t in ((f32_dir, exact), (rounded_dir, {n: v.to(torch.bfloat16) for n, v in exact.items()})):
        os.makedirs(d)
        save_file(t, os.path.join(d, "model.safetensors"))
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(TINY["A"], f)
    ids = [5, 17, 3, 250, 9, 100, 42, 7, 7, 1]
    run = lambda **kw: (lambda e: e.step([(e.alloc_slot(), ids)], "all").double().cpu().numpy())(hb.Engine.from_folder(max_tokens=128, **kw))
    as_stored = run(model_dir=f32_dir, dtype="float32")
    rounded = run(model_dir=f32_dir, dtype="float32", round_weights_to_bf16=True)
    ref_stored, ref_rounded = PlainModel(f32_dir).logits(ids).numpy(), PlainModel(rounded_dir).logits(ids).numpy()
    tol = 3e-5 * max(1.0, np.abs(ref_stored).max())
    assert np.abs(as_stored - ref_stored).max() <= tol
    assert np.abs(rounded - ref_rounded).max() <= tol
    assert np.abs(ref_stored - ref_rounded).max() > 20 * tol          # the option matters on this folder
    # the bfloat16 path with the option holds norm vectors rounded too: equal to loading the rounded folder
    a = run(model_dir=f32_dir, dtype="bfloat16", round_weights_to_bf16=True)
    b = run(model_dir=rounded_dir, dtype="bfloat16")
    assert np.array_equal(a, b)
