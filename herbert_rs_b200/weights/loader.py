"""Loading a model folder: config.json chooses the model, tensors are taken by name.

What the reference does (crates/backends/backend_common/src/loader_common.rs): classify every
tensor by its name (:413-686), convert it, assemble layers and report what a layer lacks
("layer N: missing q_proj", :847-1101), then the embedding, final norm and head (:1851-1877).
It checks no shapes and skips unknown names silently.  Here the model's parts declare their
tensors, the folder is checked against that declaration *before* anything is copied to the
device, and every fault is reported in one error: missing tensors, unexpected tensors, wrong
shapes, unusable dtypes.

Dtypes: matrices are kept in bfloat16 (the 32-bit path widens them exactly; a float32 matrix
is rounded to nearest-even for the bfloat16 path, as loader_common.rs:33-54 does); vectors
(norm weights) are kept in float32 whatever they were stored in; integer tables become int32.
The casts are kernels of this library and run on the device.

`round_weights_to_bf16=True` reproduces the reference's arithmetic on a checkpoint stored in
32-bit: it rounds *every* float tensor, norm weights included, to bfloat16 while loading
(loader_common.rs:33-54, crates/core/src/tensor.rs:46-56) and computes in float from there
(its `--backend bf16 --kv-quant f32`).  With the option the 32-bit path holds float32 matrices
whose values are bfloat16 values, and both paths hold norm vectors rounded likewise.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.base import read_config_json
from ..engine.runtime import Runtime
from ..errors import WeightError
from ..registry import config_from_json, model_class_for
from .safetensors_io import ModelFiles

_FLOAT_STORED = (torch.float32, torch.bfloat16, torch.float16)


def check_tensors(model, files) -> None:
    """Compare what the model declares with what the folder holds; raise one WeightError."""
    specs = model.param_specs()
    have = set(files.names())
    missing = sorted(n for n in specs if n not in have)
    unexpected = sorted(have - set(specs) - model.ignored_names())
    wrong_shape, wrong_dtype = [], []
    for name, ps in specs.items():
        if name not in have:
            continue
        dtype, shape = files.info(name)
        if tuple(shape) != tuple(ps.shape):
            wrong_shape.append(f"{name}: expected {list(ps.shape)}, got {list(shape)}")
        if ps.role in ("matrix", "vector") and dtype not in _FLOAT_STORED:
            wrong_dtype.append(f"{name}: stored as {dtype}, need F32, BF16 or F16")
        if ps.role == "table" and dtype not in (torch.int32, torch.int64, torch.int16, torch.int8, torch.uint8):
            wrong_dtype.append(f"{name}: stored as {dtype}, need an integer type")
    if not (missing or unexpected or wrong_shape or wrong_dtype):
        return
    lines = [f"model folder does not match {model.spec.architecture}:"]
    if missing:
        lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        head = model.spec.head_name
        if head in missing:
            lines.append(f"    ({head} is required because tie_word_embeddings is false)")
    if unexpected:
        lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong_shape:
        lines.append(f"  wrong shapes ({len(wrong_shape)}): " + "; ".join(wrong_shape))
    if wrong_dtype:
        lines.append(f"  wrong dtypes ({len(wrong_dtype)}): " + "; ".join(wrong_dtype))
    raise WeightError("\n".join(lines))


def convert(t: torch.Tensor, role: str, compute_dtype: torch.dtype, device, round_bf16: bool = False) -> torch.Tensor:
    """A stored tensor as the device tensor its role asks for (see the module's notes on dtypes)."""
    device = torch.device(device)
    if role == "table":
        return t.to(device=device, dtype=torch.int32)
    want = torch.float32 if role == "vector" else compute_dtype
    if device.type != "cuda":
        # the same rules through torch's casts: a model on the CPU can be built and filled (to read
        # its tensor list, or to test load-time fusion) but never run
        if round_bf16:
            t = t.to(torch.float32).to(torch.bfloat16)
        return t.to(device=device, dtype=want)
    from .. import ops
    src = t.to(device).contiguous()
    if src.dtype == torch.float64:
        src = src.to(torch.float32)
    return ops.cast(src, want, round_bf16)


def build_model(config_json: dict, rt: Runtime):
    """The model that config.json's architecture names, built from its configuration's spec."""
    cfg = config_from_json(config_json)
    model = model_class_for(config_json)(cfg.model_spec(), rt)
    model.config = cfg
    return model


def fill_model(model, get, rt: Runtime, round_weights_to_bf16: bool = False) -> None:
    """Give every part its tensors; `get(name)` returns a tensor on any device."""
    specs = model.param_specs()
    s = model.spec
    conv = lambda name: convert(get(name), specs[name].role, rt.dtype, rt.device, round_weights_to_bf16)  # noqa: E731
    model.load_embedding(conv(s.embed_name))
    for i, block in enumerate(model.blocks):
        prefix = model.block_prefix(i)
        model_names = [n for n in specs if n.startswith(prefix)]
        block.load({n[len(prefix):]: conv(n) for n in model_names})
    fp = model.final_norm_prefix()
    model.load_final_norm({n[len(fp):]: conv(n) for n in specs if n.startswith(fp)})
    if not s.tie_word_embeddings:
        model.load_head(conv(s.head_name))


def load_model(model_dir: str, device="cuda", dtype: torch.dtype = torch.bfloat16,
               page_size: Optional[int] = None, rt: Optional[Runtime] = None, round_weights_to_bf16: bool = False):
    """Read config.json and the safetensors of `model_dir` into a model on `device`."""
    rt = rt or Runtime(device, dtype, page_size)
    model = build_model(read_config_json(model_dir), rt)
    files = ModelFiles(model_dir)
    try:
        check_tensors(model, files)
        fill_model(model, files.tensor, rt, round_weights_to_bf16)
    finally:
        files.close()
    return model
