"""The choices between kernels that can be changed, in one record.

The reference keeps its switches in typed structs handed to the backend
(crates/core/src/backend.rs: `BackendConfig`), not in the environment; so does this library.
Every field has the value the measurements chose; a measurement script or a test assigns
another one to `herbert_rs_b200.ops.options` to take the other path.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass
class KernelOptions:
    # Products of at most 64 activation rows: "auto" picks by shape between the mma.sync kernel,
    # the streaming tcgen05 kernel and the prefill kernel; "skinny" / "stream" force one of the first two.
    decode_gemm: str = "auto"
    # A norm between two products is begun by the first and finished by the second (no norm kernel).
    shared_norm: bool = True
    # The prefill product cuts leftover output tiles into runs of k blocks shared between CTAs.
    prefill_split_tiles: bool = True
    # Head size 128, decode: norm, rotation, cache write, attention and combine in one launch.
    decode_fused: bool = True
    # Prefill attention for head sizes 64 and 128: "tcgen05", or "mma" (the mma.sync kernel for every size).
    prefill_attention: str = "tcgen05"
    # Decode attention cuts the keys so that this many CTAs stand on every SM.
    decode_ctas_per_sm: int = 2
    # ... and into at most this many key ranges per (sequence, kv head).
    decode_max_splits: int = 16
    # Programmatic dependent launch for eager steps (prompts); steps recorded as CUDA graphs never use it.
    pdl_eager: bool = True
    # The same inside recorded decode steps: 0 off, 1 every kernel, 2 only the products that load weights before they wait.
    pdl_graph: int = 0
    # Steps of 512 rows and more, heads of 128: per-head norm, rotation and cache write in the q/k/v product's epilogue.
    qkv_epilogue: bool = True
