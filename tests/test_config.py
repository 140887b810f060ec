"""Configuration and registry (no GPU)."""
import copy

import pytest

import herbert_rs_b200 as hb
from herbert_rs_b200.config import Qwen3Config
from herbert_rs_b200.errors import ConfigError
from tiny_configs import TINY


def test_reads_every_size_from_config():
    for name, c in TINY.items():
        cfg = hb.config_from_json(c)
        assert isinstance(cfg, Qwen3Config)
        assert (cfg.vocab_size, cfg.hidden_size, cfg.num_hidden_layers) == (c["vocab_size"], c["hidden_size"], c["num_hidden_layers"])
        assert cfg.q_dim == c["num_attention_heads"] * c["head_dim"]
        assert cfg.kv_dim == c["num_key_value_heads"] * c["head_dim"]
        spec = cfg.model_spec()
        assert len(spec.blocks) == c["num_hidden_layers"] and len(spec.schedule) == c["num_hidden_layers"]
        assert spec.blocks[0].mixer.qk_norm.eps == c["rms_norm_eps"]


def test_defaults_follow_reference():
    c = {k: v for k, v in TINY["A"].items() if k not in ("head_dim", "rms_norm_eps", "tie_word_embeddings", "eos_token_id", "architectures")}
    cfg = hb.config_from_json(c)
    assert cfg.head_dim == 64 // 4
    assert cfg.rms_norm_eps == 1e-5
    assert cfg.tie_word_embeddings is True
    assert cfg.eos_token_ids == (151643,)
    assert cfg.rotary_dim == cfg.head_dim
    assert abs(cfg.attn_scale - cfg.head_dim ** -0.5) < 1e-12


def test_eos_number_or_array():
    assert hb.config_from_json(TINY["A"]).eos_token_ids == (255,)
    assert hb.config_from_json(TINY["B"]).eos_token_ids == (380, 381)


def test_windows_and_options_per_layer():
    cfg = hb.config_from_json(TINY["C"])
    assert cfg.layer_windows == (None, 40, None, 40)
    assert cfg.rotary_dim == 24
    assert abs(cfg.attn_scale - 32.0 ** -0.5) < 1e-12
    spec = cfg.model_spec()
    assert [b.mixer.window for b in spec.blocks] == [None, 40, None, 40]
    c = dict(TINY["C"]); del c["layer_types"]; c["max_window_layers"] = 3
    assert hb.config_from_json(c).layer_windows == (None, None, None, 40)


def test_round_trip_through_to_dict():
    for c in TINY.values():
        cfg = hb.config_from_json(c)
        again = hb.config_from_json(cfg.to_dict())
        assert again == cfg


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                                 "num_key_value_heads", "max_position_embeddings", "rope_theta"])
def test_missing_required_key(key):
    c = dict(TINY["B"]); del c[key]
    with pytest.raises(ConfigError, match=key):
        hb.config_from_json(c)


@pytest.mark.parametrize("patch,msg", [
    ({"hidden_size": 0}, "hidden_size must be > 0"),
    ({"num_hidden_layers": 0}, "num_layers must be > 0"),
    ({"vocab_size": 0}, "vocab_size must be > 0"),
    ({"num_key_value_heads": 0}, "num_key_value_heads must be > 0"),
    ({"num_attention_heads": 6, "num_key_value_heads": 4}, "divisible"),
    ({"head_dim": 15}, "even"),
    ({"intermediate_size": 0}, "intermediate_size must be > 0"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps must be > 0"),
    ({"rope_theta": -1.0}, "rope_theta must be > 0"),
    ({"max_position_embeddings": 0}, "max_position_embeddings must be > 0"),
    ({"vocab_size": "many"}, "must be an integer"),
    ({"tie_word_embeddings": 1}, "true or false"),
    ({"attention_bias": True}, "attention_bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"num_experts": 8}, "experts"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "rope type"),
    ({"use_sliding_window": True}, "sliding_window"),
])
def test_validation_errors(patch, msg):
    c = dict(TINY["A"]); c.update(patch)
    with pytest.raises(ConfigError, match=msg):
        hb.config_from_json(c)


def test_registry_by_architecture_then_model_type():
    c = dict(TINY["A"])
    assert "Qwen3ForCausalLM" in hb.architectures()
    del c["architectures"]
    assert isinstance(hb.config_from_json(c), Qwen3Config)       # by model_type
    del c["model_type"]
    assert isinstance(hb.config_from_json(c), Qwen3Config)       # the reference's default type
    c["architectures"] = ["LlamaForCausalLM"]
    with pytest.raises(ConfigError, match="Registered: .*Qwen3ForCausalLM"):
        hb.config_from_json(c)
    with pytest.raises(ConfigError, match="unsupported architecture"):
        hb.config_from_json({"model_type": "gpt2"})


def test_register_another_architecture_from_outside():
    class Other(Qwen3Config):
        pass
    hb.register_architecture("OtherForCausalLM", Other, model_types=("other",))
    c = dict(TINY["A"]); c["architectures"] = ["OtherForCausalLM"]
    assert type(hb.config_from_json(c)) is Other


def test_unknown_part_kind_is_reported():
    from herbert_rs_b200.config import NormSpec
    with pytest.raises(ConfigError, match="no norm registered"):
        hb.build_part("norm", NormSpec(8, 1e-5, kind="layernorm_of_mars"), rt=None)


def test_backend_names():
    text = hb.available_backends_help()
    assert "cuda-bf16" in text and "cuda-fp32" in text and "auto" in text
    with pytest.raises(hb.BackendError, match="unknown backend 'tpu'"):
        hb.resolve_backend("tpu")
