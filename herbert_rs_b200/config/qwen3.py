"""Typed configuration of the dense Qwen3 decoder, read from its config.json keys.

Keys, defaults and validation follow the reference's `Config::from_json` and
`Config::validate` (crates/core/src/config.rs:183-255, 366-441, 490-694):

* required: vocab_size, hidden_size, num_hidden_layers, num_attention_heads,
  num_key_value_heads, max_position_embeddings, rope_theta (or rope_parameters.rope_theta);
* head_dim defaults to hidden_size / num_attention_heads (config.rs:496-498);
* rms_norm_eps defaults to 1e-5 (config.rs:583-585);
* tie_word_embeddings defaults to true when absent (config.rs:199-202);
* eos_token_id is a number or an array (config.rs:266-274); the reference keeps the
  first element and falls back to 151643 (config.rs:285-287); here every element is a
  stop token and the fallback is the same;
* partial_rotary_factor (top level or inside rope_parameters) gives the rotated width
  (config.rs:516-525); query_pre_attn_scalar gives scale = 1/sqrt(s) (config.rs:645-646).

The reference never reads sliding_window / use_sliding_window / max_window_layers /
layer_types, attention_bias or hidden_act.  This library does not ignore them silently:
windows are honoured layer by layer, and values it cannot serve are refused.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

from ..errors import ConfigError
from .base import Reader
from .specs import (
    AttentionSpec,
    BlockSpec,
    ModelSpec,
    NormSpec,
    PositionSpec,
    SwiGLUSpec,
    identity_schedule,
)

DEFAULT_EOS_TOKEN = 151643  # crates/core/src/config.rs:285-287


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    rope_theta: float
    rms_norm_eps: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    eos_token_ids: tuple
    rotary_dim: int
    attn_scale: float
    layer_windows: tuple  # per layer: None (all keys) or the window length
    model_type: str = "qwen3"

    # -- derived sizes (crates/core/src/config.rs:305-319) --------------------------------
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def num_kv_groups(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    # -- reading -----------------------------------------------------------------------
    @classmethod
    def from_dict(cls, obj: dict) -> "Qwen3Config":
        r = Reader(obj)
        model_type = r.string("model_type", "qwen3")
        vocab = r.integer("vocab_size")
        hidden = r.integer("hidden_size")
        layers = r.integer("num_hidden_layers")
        heads = r.integer("num_attention_heads")
        kv_heads = r.integer("num_key_value_heads")
        max_pos = r.integer("max_position_embeddings")
        if heads <= 0:
            raise ConfigError("num_attention_heads must be > 0")
        head_dim = r.integer("head_dim", None)
        if head_dim is None:
            head_dim = hidden // heads
        inter = r.integer("intermediate_size", 0)
        eps = r.number("rms_norm_eps", 1e-5)
        tie = r.boolean("tie_word_embeddings", True)

        rope_parameters = r.raw("rope_parameters")
        rope_scaling = r.raw("rope_scaling")
        theta = r.number("rope_theta", None)
        if theta is None and isinstance(rope_parameters, dict):
            t = rope_parameters.get("rope_theta")
            if isinstance(t, (int, float)) and not isinstance(t, bool):
                theta = float(t)
        if theta is None:
            raise ConfigError("missing rope_theta (or rope_parameters.rope_theta)")

        prf = r.number("partial_rotary_factor", None)
        if prf is None and isinstance(rope_parameters, dict):
            t = rope_parameters.get("partial_rotary_factor")
            if isinstance(t, (int, float)) and not isinstance(t, bool):
                prf = float(t)
        if prf is None:
            prf = 1.0
        rotary_dim = int(head_dim * prf)

        for name, params in (("rope_parameters", rope_parameters), ("rope_scaling", rope_scaling)):
            if isinstance(params, dict):
                kind = params.get("rope_type", params.get("type"))
                factor = params.get("factor", 1.0)
                if kind not in (None, "default") and not (kind == "linear" and factor <= 1.0):
                    raise ConfigError(
                        f"{name}: rope type {kind!r} is not supported (only unscaled rotary positions)"
                    )

        qpas = r.number("query_pre_attn_scalar", None)
        if qpas is not None and qpas <= 0:
            raise ConfigError("query_pre_attn_scalar must be > 0")
        scale = 1.0 / math.sqrt(qpas) if qpas is not None else (
            1.0 / math.sqrt(head_dim) if head_dim > 0 else 0.0)

        eos_raw = r.raw("eos_token_id")
        eos: tuple
        if isinstance(eos_raw, bool):
            eos = ()
        elif isinstance(eos_raw, int):
            eos = (eos_raw,)
        elif isinstance(eos_raw, list):
            eos = tuple(int(v) for v in eos_raw if isinstance(v, int) and not isinstance(v, bool))
        else:
            eos = ()
        if not eos:
            eos = (DEFAULT_EOS_TOKEN,)

        if r.boolean("attention_bias", False):
            raise ConfigError("attention_bias=true is not supported: Qwen3 projections carry no bias")
        act = r.string("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act {act!r} is not supported: the feed-forward is SwiGLU (silu)")
        if r.has("num_experts") or r.has("num_local_experts"):
            raise ConfigError("num_experts is set: routed experts are not part of the dense Qwen3 decoder")

        # Windows, layer by layer.
        windows: list = [None] * max(layers, 0)
        if r.boolean("use_sliding_window", False):
            window = r.integer("sliding_window", None)
            if window is None or window <= 0:
                raise ConfigError("use_sliding_window is true but sliding_window is not a positive integer")
            layer_types = r.raw("layer_types")
            if layer_types is not None:
                if not isinstance(layer_types, list) or len(layer_types) != layers:
                    raise ConfigError("layer_types must list one entry per layer")
                for i, t in enumerate(layer_types):
                    if t == "sliding_attention":
                        windows[i] = window
                    elif t != "full_attention":
                        raise ConfigError(f"layer_types[{i}] = {t!r} is not a known attention type")
            else:
                first = r.integer("max_window_layers", layers)
                for i in range(layers):
                    if i >= first:
                        windows[i] = window

        cfg = cls(
            vocab_size=vocab, hidden_size=hidden, num_hidden_layers=layers,
            num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
            intermediate_size=inter, rope_theta=float(theta), rms_norm_eps=float(eps),
            max_position_embeddings=max_pos, tie_word_embeddings=tie, eos_token_ids=eos,
            rotary_dim=rotary_dim, attn_scale=scale, layer_windows=tuple(windows),
            model_type=model_type,
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        """Same checks, same order and wording as crates/core/src/config.rs:366-407."""
        if self.hidden_size <= 0:
            raise ConfigError("hidden_size must be > 0")
        if self.num_hidden_layers <= 0:
            raise ConfigError("num_layers must be > 0")
        if self.vocab_size <= 0:
            raise ConfigError("vocab_size must be > 0")
        if self.num_attention_heads <= 0:
            raise ConfigError("num_attention_heads must be > 0")
        if self.num_key_value_heads <= 0:
            raise ConfigError("num_key_value_heads must be > 0")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be divisible by "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim <= 0 or self.head_dim % 2 != 0:
            raise ConfigError(f"head_dim ({self.head_dim}) must be > 0 and even (required by RoPE)")
        if self.intermediate_size <= 0:
            raise ConfigError("intermediate_size must be > 0")
        if not self.rms_norm_eps > 0.0:
            raise ConfigError("rms_norm_eps must be > 0")
        if not self.rope_theta > 0.0:
            raise ConfigError("rope_theta must be > 0")
        if self.max_position_embeddings <= 0:
            raise ConfigError("max_position_embeddings must be > 0")
        if self.rotary_dim <= 0 or self.rotary_dim % 2 != 0 or self.rotary_dim > self.head_dim:
            raise ConfigError(
                f"rotated width ({self.rotary_dim}) must be even and in 2..head_dim ({self.head_dim})")

    # -- writing -----------------------------------------------------------------------
    def to_dict(self) -> dict:
        """The config.json that `from_dict` reads back to an equal configuration."""
        d = {
            "architectures": ["Qwen3ForCausalLM"],
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "rope_theta": self.rope_theta,
            "rms_norm_eps": self.rms_norm_eps,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "eos_token_id": list(self.eos_token_ids) if len(self.eos_token_ids) != 1 else self.eos_token_ids[0],
            "hidden_act": "silu",
            "attention_bias": False,
        }
        if self.rotary_dim != self.head_dim:
            d["partial_rotary_factor"] = self.rotary_dim / self.head_dim
        if abs(self.attn_scale - 1.0 / math.sqrt(self.head_dim)) > 1e-12:
            d["query_pre_attn_scalar"] = 1.0 / (self.attn_scale * self.attn_scale)
        if any(w is not None for w in self.layer_windows):
            d["use_sliding_window"] = True
            d["sliding_window"] = next(w for w in self.layer_windows if w is not None)
            d["layer_types"] = ["full_attention" if w is None else "sliding_attention"
                                for w in self.layer_windows]
        return d

    # -- the layer list ------------------------------------------------------------------
    def model_spec(self) -> ModelSpec:
        """Layers as data: every layer is attention + SwiGLU in a pre-norm block
        (crates/backends/backend_common/src/generic_layer.rs:1131-1328)."""
        norm = NormSpec(self.hidden_size, self.rms_norm_eps)
        head_norm = NormSpec(self.head_dim, self.rms_norm_eps)
        rope = PositionSpec(self.head_dim, self.rotary_dim, self.rope_theta, self.max_position_embeddings)
        ffn = SwiGLUSpec(self.hidden_size, self.intermediate_size)
        blocks = []
        for i in range(self.num_hidden_layers):
            mixer = AttentionSpec(
                hidden_size=self.hidden_size, num_heads=self.num_attention_heads,
                num_kv_heads=self.num_key_value_heads, head_dim=self.head_dim,
                scale=self.attn_scale, qk_norm=head_norm, position=rope,
                window=self.layer_windows[i])
            blocks.append(BlockSpec(mixer=mixer, ffn=ffn, norm1=norm, norm2=norm))
        return ModelSpec(
            architecture="Qwen3ForCausalLM", vocab_size=self.vocab_size, hidden_size=self.hidden_size,
            blocks=tuple(blocks), schedule=identity_schedule(self.num_hidden_layers),
            final_norm=norm, tie_word_embeddings=self.tie_word_embeddings,
            max_position=self.max_position_embeddings, stop_token_ids=tuple(self.eos_token_ids))
