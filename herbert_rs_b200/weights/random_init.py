"""Random weights from a configuration and a seed.

The reference has no such mode (it only loads checkpoints); this one exists so that tests and
measurements need no download.  Distributions: matrices N(0, 0.02); norm weights 1 + N(0, 0.1).
Element i of tensor `name` is a function of (seed, name, i) alone (`counter_rng`): it does not
depend on which other tensors exist, on the order in which they are made, or on whether the CPU
or a kernel of this library on the GPU made it: both give the same bytes.  So a model made
directly on the device is the model that `write_random_model` writes for the same seed.  Values
are rounded to bfloat16 and stored as BF16, so the 32-bit path and the bfloat16 path read
identical weights.
"""

from __future__ import annotations

import json
import os
from typing import Dict

import torch

from ..engine.runtime import Runtime
from ..registry import config_from_json
from . import counter_rng
from .loader import build_model, fill_model
from .safetensors_io import save_stream

_INIT = {"normal": (0.0, 0.02), "ones_noise": (1.0, 0.1)}


def random_tensor(name: str, ps, seed: int, device="cpu") -> torch.Tensor:
    """The tensor `name` of a random model, as bfloat16 values (int32 for tables), on `device`."""
    device = torch.device(device)
    if ps.role == "table":
        return torch.zeros(ps.shape, dtype=torch.int32, device=device)
    if ps.init == "zeros":
        return torch.zeros(ps.shape, dtype=torch.bfloat16, device=device)
    mean, std = _INIT[ps.init]
    key = counter_rng.tensor_key(seed, name)
    n = 1
    for d in ps.shape:
        n *= int(d)
    if device.type == "cuda":
        from .. import ops
        t = torch.empty(ps.shape, dtype=torch.bfloat16, device=device)
        ops.rng_normal(t, key, mean, std)
        return t
    return counter_rng.normal(key, n, mean, std, torch.bfloat16).view(tuple(ps.shape))


def random_tensors(model, seed: int, device="cpu") -> Dict[str, torch.Tensor]:
    return {name: random_tensor(name, ps, seed, device) for name, ps in model.param_specs().items()}


def write_random_model(config_json: dict, out_dir: str, seed: int = 0, device="cpu") -> str:
    """Write `out_dir/config.json` and `out_dir/model.safetensors` for random weights.  `device`
    is where the numbers are made ("cuda": by the library's kernel, much faster for large models);
    the file is the same either way."""
    cfg = config_from_json(config_json)
    model = build_model(config_json, Runtime("cpu", torch.bfloat16))
    os.makedirs(out_dir, exist_ok=True)
    full = dict(cfg.to_dict()) if hasattr(cfg, "to_dict") else dict(config_json)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(full, f, indent=1)
    specs = model.param_specs()
    entries = [(name, torch.int32 if ps.role == "table" else torch.bfloat16, tuple(ps.shape),
                (lambda name=name, ps=ps: random_tensor(name, ps, seed, device))) for name, ps in specs.items()]
    save_stream(entries, os.path.join(out_dir, "model.safetensors"), metadata={"format": "pt", "seed": seed})
    return out_dir


def random_model(config_json: dict, seed: int, rt: Runtime):
    """A model with random weights made directly on the runtime's device (no folder): the same
    weights, bit for bit, as the folder `write_random_model` writes for this seed."""
    model = build_model(config_json, rt)
    specs = model.param_specs()
    fill_model(model, lambda name: random_tensor(name, specs[name], seed, rt.device), rt)
    return model
