"""Random weights from a configuration and a seed.

The reference has no such mode (it only loads checkpoints); this one exists so that tests and
measurements need no download.  Distributions: matrices N(0, 0.02); norm weights 1 + N(0, 0.1).
Every tensor has its own generator seeded from (seed, tensor name), so a tensor's values do not
depend on which other tensors exist or in which order they are made.  Values are rounded to
bfloat16 and stored as BF16, so the 32-bit path and the bfloat16 path read identical weights.
"""

from __future__ import annotations

import hashlib
import json
import os
from typing import Dict

import torch

from ..engine.runtime import Runtime
from ..models.decoder import DecoderModel
from ..registry import config_from_json
from .loader import build_model, fill_model
from .safetensors_io import save_file


def _seed_for(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(name: str, ps, seed: int, device="cpu") -> torch.Tensor:
    """The tensor `name` of a random model, as bfloat16 values (int32 for tables)."""
    g = torch.Generator(device=device)
    g.manual_seed(_seed_for(seed, name))
    if ps.role == "table":
        return torch.zeros(ps.shape, dtype=torch.int32, device=device)
    if ps.init == "zeros":
        t = torch.zeros(ps.shape, dtype=torch.float32, device=device)
    else:
        t = torch.randn(ps.shape, generator=g, dtype=torch.float32, device=device)
        t = 1.0 + 0.1 * t if ps.init == "ones_noise" else 0.02 * t
    return t.to(torch.bfloat16)


def random_tensors(model: DecoderModel, seed: int, device="cpu") -> Dict[str, torch.Tensor]:
    return {name: random_tensor(name, ps, seed, device) for name, ps in model.param_specs().items()}


def write_random_model(config_json: dict, out_dir: str, seed: int = 0) -> str:
    """Write `out_dir/config.json` and `out_dir/model.safetensors` for random weights."""
    cfg = config_from_json(config_json)
    model = DecoderModel(cfg.model_spec(), Runtime("cpu", torch.bfloat16))
    os.makedirs(out_dir, exist_ok=True)
    full = dict(cfg.to_dict()) if hasattr(cfg, "to_dict") else dict(config_json)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(full, f, indent=1)
    save_file(random_tensors(model, seed), os.path.join(out_dir, "model.safetensors"),
              metadata={"format": "pt", "seed": seed})
    return out_dir


def random_model(config_json: dict, seed: int, rt: Runtime) -> DecoderModel:
    """A model with random weights made directly on the runtime's device (no folder).

    Uses the device's own generator, so values differ from `write_random_model`'s for the same
    seed; meant for measurements at sizes where writing a folder would only cost time."""
    model = build_model(config_json, rt)
    specs = model.param_specs()
    fill_model(model, lambda name: random_tensor(name, specs[name], seed, rt.device), rt)
    return model
