"""Size-and-constant records ("specs") from which parts are built.

A spec is plain data: it says which kind of part stands at a place and with which
sizes and constants.  An architecture's configuration produces a `ModelSpec`; the
part registry (`herbert_rs_b200.registry`) turns every spec into a part by its
`kind`.  No spec and no part knows which model it belongs to.

The reference keeps the same facts as fields of its generic parts
(crates/backends/backend_common/src/generic_attention/mod.rs:27-59 for the mixer,
generic_mlp.rs:20-28 for the feed-forward, generic_layer.rs:705-719 for the block);
here they are separated from the parts so that a layer list is data.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence


@dataclass(frozen=True)
class NormSpec:
    """A normalisation over the last axis.  kind "rmsnorm": y = x / sqrt(mean(x^2) + eps) * w."""

    dim: int
    eps: float
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class PositionSpec:
    """A position encoding applied inside a mixer.  kind "rope": half-split rotary pairs."""

    head_dim: int
    rotary_dim: int
    theta: float
    max_position: int
    kind: str = "rope"


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query softmax attention over cached keys and values."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    qk_norm: Optional[NormSpec] = None
    position: Optional[PositionSpec] = None
    window: Optional[int] = None  # None: every earlier key; n: the last n keys (itself included)
    kind: str = "attention"


@dataclass(frozen=True)
class SwiGLUSpec:
    """Dense gated feed-forward: down(silu(gate(x)) * up(x))."""

    hidden_size: int
    intermediate_size: int
    kind: str = "swiglu"


@dataclass(frozen=True)
class BlockSpec:
    """One layer: how a mixer, a feed-forward and their norms are arranged.

    kind "prenorm": h = x + mixer(norm1(x)); out = h + ffn(norm2(h)).
    `names` maps the block's local part names to the sub-prefixes used in tensor names.
    """

    mixer: object
    ffn: object
    norm1: NormSpec
    norm2: NormSpec
    kind: str = "prenorm"
    names: tuple = (
        ("norm1", "input_layernorm"),
        ("mixer", "self_attn"),
        ("norm2", "post_attention_layernorm"),
        ("ffn", "mlp"),
    )


@dataclass(frozen=True)
class ScheduleStep:
    """One entry of the execution order.

    `layer` indexes `ModelSpec.blocks`; a layer may be named by several steps (its weights
    are then used several times, each step with a cache entry of its own).  A step with
    `reads_cache_of = k` stores nothing: its mixer reads what step k (an earlier step) stored.
    """

    layer: int
    reads_cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    """Everything the generic decoder needs: table sizes, layers, order, output head."""

    architecture: str
    vocab_size: int
    hidden_size: int
    blocks: Sequence[BlockSpec]
    schedule: Sequence[ScheduleStep]
    final_norm: NormSpec
    tie_word_embeddings: bool
    max_position: int
    stop_token_ids: tuple = ()
    layer_prefix: str = "model.layers.{i}."
    embed_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm.weight"
    head_name: str = "lm_head.weight"
    # How many numbers place a token: 1 for a position in a sequence.  An encoding that needs
    # more (rows and columns of an image, say) raises this; the step then carries that many position
    # rows per token, which the caller may give per sequence (Engine.step(..., positions=...)) and
    # which default to the token's index in its sequence in every component.
    position_components: int = 1
    extra: dict = field(default_factory=dict)     # free for an architecture's own model class


def identity_schedule(n: int) -> tuple:
    """Every layer once, in order, each with its own cache entry."""
    return tuple(ScheduleStep(i) for i in range(n))
