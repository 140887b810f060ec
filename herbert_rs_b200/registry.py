"""Two registries: architectures by name, and parts by kind.

Architectures.  The reference dispatches on the `model_type` string
(crates/core/src/config.rs:93-103) and reports an unknown one with the list of those it
supports (config.rs:500-506).  Here the key is config.json's `architectures[0]`, with
`model_type` as the fallback, and the value is the typed configuration class whose
`model_spec()` describes the layers.

Parts.  A spec's `kind` string selects the class that is built from it.  The reference
does this with enums inside its generic layer (`LayerBlock`, `GenericFFN`, `NormType`:
crates/backends/backend_common/src/generic_layer.rs:698-702, generic_moe.rs:38-41); a
table keeps it open, so a new mixer, feed-forward, norm, position encoding or block is
registered from outside without touching these files.
"""

from __future__ import annotations

from typing import Callable, Dict

from .errors import ConfigError

_ARCHITECTURES: Dict[str, type] = {}
_MODEL_CLASSES: Dict[str, type] = {}
_MODEL_TYPES: Dict[str, str] = {}
_DEFAULT_ARCHITECTURE: list = []
_PARTS: Dict[str, Dict[str, Callable]] = {
    "mixer": {}, "ffn": {}, "norm": {}, "position": {}, "block": {},
}


def register_architecture(name: str, config_cls: type, model_types: tuple = (), model_cls: type = None,
                          default: bool = False) -> None:
    """Register `config_cls` (with `from_dict(dict)` and `model_spec()`) under an architecture name.

    `model_cls(spec, rt)` is the class built from the spec (the generic decoder when None): an
    architecture whose top level differs (scaled embeddings, a cap on the logits, a second head)
    brings its own.  `default=True` makes this the architecture of a config.json that names neither
    `architectures` nor `model_type` (the reference defaults `model_type` to "qwen3",
    crates/core/src/config.rs:184-185, 261-263)."""
    _ARCHITECTURES[name] = config_cls
    if model_cls is not None:
        _MODEL_CLASSES[name] = model_cls
    else:
        _MODEL_CLASSES.pop(name, None)
    for mt in model_types:
        _MODEL_TYPES[mt] = name
    if default:
        _DEFAULT_ARCHITECTURE[:] = [name]


def architectures() -> list:
    return sorted(_ARCHITECTURES)


def architecture_for(config_json: dict) -> str:
    """The registered architecture name chosen by config.json's `architectures`, else `model_type`,
    else the registered default."""
    archs = config_json.get("architectures")
    names = [a for a in archs if isinstance(a, str)] if isinstance(archs, list) else []
    for a in names:
        if a in _ARCHITECTURES:
            return a
    mt = config_json.get("model_type")
    if not names and isinstance(mt, str) and mt in _MODEL_TYPES:
        return _MODEL_TYPES[mt]
    if not names and mt is None and _DEFAULT_ARCHITECTURE and _DEFAULT_ARCHITECTURE[0] in _ARCHITECTURES:
        return _DEFAULT_ARCHITECTURE[0]
    asked = names[0] if names else mt
    raise ConfigError(
        f"unsupported architecture: {asked!r}. Registered: {', '.join(architectures()) or '(none)'}")


def config_class_for(config_json: dict) -> type:
    return _ARCHITECTURES[architecture_for(config_json)]


def model_class_for(config_json: dict) -> type:
    """The model class of config.json's architecture (the generic decoder unless it brought its own)."""
    name = architecture_for(config_json)
    if name in _MODEL_CLASSES:
        return _MODEL_CLASSES[name]
    from .models.decoder import DecoderModel
    return DecoderModel


def config_from_json(config_json: dict):
    return config_class_for(config_json).from_dict(config_json)


def register_part(role: str, kind: str, factory: Callable) -> None:
    """Register a part class for a spec kind.  role: mixer | ffn | norm | position | block."""
    if role not in _PARTS:
        raise ValueError(f"unknown part role {role!r}")
    _PARTS[role][kind] = factory


def part_factory(role: str, kind: str) -> Callable:
    try:
        return _PARTS[role][kind]
    except KeyError:
        known = ", ".join(sorted(_PARTS.get(role, {}))) or "(none)"
        raise ConfigError(f"no {role} registered for kind {kind!r}; registered: {known}") from None


def build_part(role: str, spec, **kw):
    """Build the part a spec describes.  Every spec carries its `kind`."""
    return part_factory(role, spec.kind)(spec, **kw)
