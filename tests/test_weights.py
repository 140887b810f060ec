"""Safetensors by name, the one error that lists every fault, and random folders (no GPU)."""
import json
import os
import struct

import pytest
import torch

import herbert_rs_b200 as hb
from herbert_rs_b200.engine.runtime import Runtime
from herbert_rs_b200.errors import SafeTensorsError, WeightError
from herbert_rs_b200.models.decoder import DecoderModel
from herbert_rs_b200.weights import ModelFiles, check_tensors, random_tensors, save_file, write_random_model
from herbert_rs_b200.weights.loader import build_model, convert, fill_model
from tiny_configs import TINY


def _model(cfg):
    return build_model(cfg, Runtime("cpu", torch.bfloat16))


def _folder(tmp_path, cfg, tensors):
    d = tmp_path / "m"
    d.mkdir(exist_ok=True)
    (d / "config.json").write_text(json.dumps(cfg))
    save_file(tensors, str(d / "model.safetensors"))
    return str(d)


def test_random_folder_round_trip(tmp_path):
    for name, cfg in TINY.items():
        d = write_random_model(cfg, str(tmp_path / name), seed=3)
        assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
        m = _model(json.load(open(os.path.join(d, "config.json"))))
        files = ModelFiles(d)
        check_tensors(m, files)
        specs = m.param_specs()
        assert set(files.names()) == set(specs)
        for n, ps in specs.items():
            dt, shape = files.info(n)
            assert dt == torch.bfloat16 and tuple(shape) == tuple(ps.shape)
        files.close()


def test_random_weights_depend_only_on_seed_and_name(tmp_path):
    m = _model(TINY["B"])
    a, b, c = random_tensors(m, 5), random_tensors(m, 5), random_tensors(m, 6)
    for n in a:
        assert torch.equal(a[n], b[n])
    assert not torch.equal(a["model.layers.0.mlp.up_proj.weight"], c["model.layers.0.mlp.up_proj.weight"])
    w = a["model.layers.1.self_attn.k_proj.weight"].float()
    assert abs(w.std().item() - 0.02) < 0.003 and abs(w.mean().item()) < 0.003
    nw = a["model.layers.1.input_layernorm.weight"].float()
    assert abs(nw.mean().item() - 1.0) < 0.05 and 0.05 < nw.std().item() < 0.15


def test_tensor_names_are_the_checkpoint_names():
    names = set(_model(TINY["B"]).param_specs())
    for n in ["model.embed_tokens.weight", "model.norm.weight", "lm_head.weight",
              "model.layers.2.input_layernorm.weight", "model.layers.2.post_attention_layernorm.weight",
              "model.layers.0.self_attn.q_proj.weight", "model.layers.0.self_attn.k_proj.weight",
              "model.layers.0.self_attn.v_proj.weight", "model.layers.0.self_attn.o_proj.weight",
              "model.layers.0.self_attn.q_norm.weight", "model.layers.0.self_attn.k_norm.weight",
              "model.layers.1.mlp.gate_proj.weight", "model.layers.1.mlp.up_proj.weight",
              "model.layers.1.mlp.down_proj.weight"]:
        assert n in names
    assert "lm_head.weight" not in _model(TINY["A"]).param_specs()   # tied


def test_one_error_lists_missing_unexpected_and_shapes(tmp_path):
    cfg = TINY["B"]
    t = random_tensors(_model(cfg), 1)
    del t["model.layers.1.self_attn.q_norm.weight"]
    del t["lm_head.weight"]
    t["model.layers.0.mlp.gate_proj.weight"] = torch.zeros(10, 96, dtype=torch.bfloat16)
    t["model.layers.9.mlp.extra.weight"] = torch.zeros(3, dtype=torch.bfloat16)
    t["model.norm.weight"] = torch.zeros(96, dtype=torch.int32)
    d = _folder(tmp_path, cfg, t)
    with pytest.raises(WeightError) as e:
        check_tensors(_model(cfg), ModelFiles(d))
    msg = str(e.value)
    assert "missing tensors (2)" in msg and "model.layers.1.self_attn.q_norm.weight" in msg and "lm_head.weight" in msg
    assert "tie_word_embeddings is false" in msg
    assert "unexpected tensors (1): model.layers.9.mlp.extra.weight" in msg
    assert "model.layers.0.mlp.gate_proj.weight: expected [224, 96], got [10, 96]" in msg
    assert "wrong dtypes (1)" in msg and "model.norm.weight" in msg


def test_tied_model_ignores_a_stored_head(tmp_path):
    cfg = TINY["A"]
    t = random_tensors(_model(cfg), 1)
    t["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)
    check_tensors(_model(cfg), ModelFiles(_folder(tmp_path, cfg, t)))


def test_dtype_rules():
    f32 = torch.tensor([1.0 + 2 ** -8, 1.0 + 3 * 2 ** -8], dtype=torch.float32)  # two ties
    # matrices: float32 -> bfloat16 rounds to nearest even (core/src/tensor.rs:46-56)
    assert convert(f32, "matrix", torch.bfloat16, "cpu").tolist() == [1.0, 1.015625]
    assert convert(f32, "matrix", torch.float32, "cpu").dtype == torch.float32
    # vectors stay 32-bit on both paths; bfloat16 ones widen exactly
    assert torch.equal(convert(f32, "vector", torch.bfloat16, "cpu"), f32)
    b = torch.tensor([0.3], dtype=torch.bfloat16)
    assert convert(b, "vector", torch.bfloat16, "cpu").dtype == torch.float32
    assert convert(b, "vector", torch.bfloat16, "cpu").item() == b.float().item()
    assert convert(torch.tensor([3], dtype=torch.int64), "table", torch.bfloat16, "cpu").dtype == torch.int32


def test_fill_model_fuses_projections(tmp_path):
    cfg = TINY["C"]
    m = _model(cfg)
    t = random_tensors(m, 2)
    fill_model(m, lambda n: t[n], m.rt)
    mixer, ffn = m.blocks[0].mixer, m.blocks[0].ffn
    assert mixer.wqkv.shape == (6 * 48 + 2 * 3 * 48, 80)
    assert torch.equal(mixer.wqkv[: 6 * 48], t["model.layers.0.self_attn.q_proj.weight"])
    assert ffn.interleave == 0 and ffn.wgu.shape == (2 * 172, 80)     # 172 is no multiple of 8
    m2 = _model(TINY["B"]); t2 = random_tensors(m2, 2); fill_model(m2, lambda n: t2[n], m2.rt)
    f2 = m2.blocks[1].ffn
    assert f2.interleave == 8
    assert torch.equal(f2.wgu[16:24], t2["model.layers.1.mlp.gate_proj.weight"][8:16])
    assert torch.equal(f2.wgu[24:32], t2["model.layers.1.mlp.up_proj.weight"][8:16])
    assert m.head is not m.embed and _model(TINY["A"]).spec.tie_word_embeddings


def test_sharded_folder(tmp_path):
    cfg = TINY["A"]
    t = random_tensors(_model(cfg), 4)
    names = sorted(t)
    d = tmp_path / "s"; d.mkdir()
    (d / "config.json").write_text(json.dumps(cfg))
    half = len(names) // 2
    save_file({n: t[n] for n in names[:half]}, str(d / "model-00001-of-00002.safetensors"))
    save_file({n: t[n] for n in names[half:]}, str(d / "model-00002-of-00002.safetensors"))
    wm = {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors") for i, n in enumerate(names)}
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    files = ModelFiles(str(d))
    check_tensors(_model(cfg), files)
    assert torch.equal(files.tensor(names[-1]), t[names[-1]])
    wm["model.ghost.weight"] = "model-00001-of-00002.safetensors"
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    with pytest.raises(SafeTensorsError, match="listed in the index but missing"):
        ModelFiles(str(d))


def test_container_faults(tmp_path):
    cfg = TINY["A"]
    d = write_random_model(cfg, str(tmp_path / "ok"), seed=1)
    p = os.path.join(d, "model.safetensors")
    raw = open(p, "rb").read()
    bad = tmp_path / "bad"; bad.mkdir()
    def put(b):
        open(bad / "model.safetensors", "wb").write(b)
    put(raw[: len(raw) - 100])
    with pytest.raises(SafeTensorsError, match="truncated"):
        ModelFiles(str(bad))
    put(raw[:5])
    with pytest.raises(SafeTensorsError, match="truncated"):
        ModelFiles(str(bad))
    put(struct.pack("<Q", 10) + b"not json!!" + b"\0" * 16)
    with pytest.raises(SafeTensorsError, match="not valid JSON"):
        ModelFiles(str(bad))
    hdr = json.dumps({"x": {"dtype": "F8_E4M3", "shape": [2], "data_offsets": [0, 2]}}).encode()
    put(struct.pack("<Q", len(hdr)) + hdr + b"\0\0")
    with pytest.raises(SafeTensorsError, match="unsupported dtype"):
        ModelFiles(str(bad))
    hdr = json.dumps({"x": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}).encode()
    put(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 4)
    with pytest.raises(SafeTensorsError, match="needs 8 bytes"):
        ModelFiles(str(bad))
    with pytest.raises(SafeTensorsError, match="no model.safetensors"):
        ModelFiles(str(tmp_path))


def test_our_writer_is_read_by_the_safetensors_package(tmp_path):
    st = pytest.importorskip("safetensors.torch")
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(4, dtype=torch.float32)}
    save_file(t, str(tmp_path / "x.safetensors"))
    back = st.load_file(str(tmp_path / "x.safetensors"))
    assert torch.equal(back["a"], t["a"]) and torch.equal(back["b"], t["b"])


def test_counter_rng_is_addressed_by_element_and_looks_normal():
    from herbert_rs_b200.weights import counter_rng as R
    key = R.tensor_key(3, "model.layers.0.mlp.down_proj.weight")
    assert key != R.tensor_key(4, "model.layers.0.mlp.down_proj.weight") != R.tensor_key(3, "model.layers.1.mlp.down_proj.weight")
    whole = R.normal(key, 300000, 0.0, 1.0)
    assert torch.equal(whole[1234:1234 + 5000], R.normal(key, 5000, 0.0, 1.0, start=1234))     # any piece alone
    assert torch.equal(R.normal(key, 1000, 1.0, 0.1, torch.bfloat16).float(),
                       (1.0 + 0.1 * whole[:1000]).to(torch.bfloat16).float())
    z = whole.double()
    assert abs(z.mean()) < 0.01 and abs(z.std() - 1) < 0.01 and 2.9 < (z ** 4).mean() < 3.1
    assert 0.0020 < (z.abs() > 3).double().mean() < 0.0034 and z.abs().max() < 6.0
    other = R.normal(R.tensor_key(3, "x"), 300000, 0.0, 1.0).double()
    assert abs((z * other).mean()) < 0.01                                                     # streams do not follow each other


def test_a_tensor_of_a_random_model_depends_on_seed_and_name_only(tmp_path):
    import herbert_rs_b200 as hb
    from herbert_rs_b200.weights import ModelFiles
    a, b = dict(TINY["A"]), dict(TINY["A"])
    b["num_hidden_layers"] = 3                      # another tensor list: the shared names keep their bytes
    hb.write_random_model(a, str(tmp_path / "a"), seed=9)
    hb.write_random_model(b, str(tmp_path / "b"), seed=9)
    fa, fb = ModelFiles(str(tmp_path / "a")), ModelFiles(str(tmp_path / "b"))
    for n in fa.names():
        assert torch.equal(fa.tensor(n).view(torch.int16), fb.tensor(n).view(torch.int16))
    w = fa.tensor("model.layers.1.input_layernorm.weight").float()
    assert abs(w.mean() - 1) < 0.05 and 0.05 < w.std() < 0.15
