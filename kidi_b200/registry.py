"""One registry from an architecture's name to its model.

The reference keeps an array of descriptors {type, validate_config, create} and
finds a model by the normalised `model_type` (src/kidi/model/registry.cpp:29-95;
unknown types are UNSUPPORTED, src/kidi/checkpoint/config.cpp:260-264). Here an
architecture registers a typed configuration class and a function that turns a
configuration into a `ModelSpec`; config.json selects it through
`architectures[0]`, or through `model_type` when that key is absent.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Callable, Dict, Mapping, Optional, Tuple

from .errors import invalid_manifest, unsupported
from .parts.spec import ModelSpec


@dataclasses.dataclass(frozen=True)
class Architecture:
    name: str
    config_type: type                      # has from_dict(mapping) and to_dict()
    build_spec: Callable[[Any], ModelSpec]
    aliases: Tuple[str, ...] = ()


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_type: type, build_spec: Callable[[Any], ModelSpec],
                          aliases: Tuple[str, ...] = ()) -> Architecture:
    entry = Architecture(name, config_type, build_spec, tuple(aliases))
    for key in (name, *aliases):
        _ARCHITECTURES[key] = entry
    return entry


def find_architecture(name: str) -> Optional[Architecture]:
    _load_builtin()
    return _ARCHITECTURES.get(name)


def registered_architectures() -> Tuple[str, ...]:
    _load_builtin()
    return tuple(sorted({entry.name for entry in _ARCHITECTURES.values()}))


def resolve_architecture(config: Mapping[str, Any]) -> Architecture:
    """Chooses the architecture a config.json names."""
    _load_builtin()
    names = config.get("architectures")
    key = None
    if isinstance(names, (list, tuple)) and names and isinstance(names[0], str):
        key = names[0]
    elif names is not None:
        raise invalid_manifest("'architectures' must be a non-empty list of strings")
    if key is None or key not in _ARCHITECTURES:
        model_type = config.get("model_type")
        if model_type is not None and not isinstance(model_type, str):
            raise invalid_manifest("'model_type' must be a string")
        if isinstance(model_type, str) and (model_type in _ARCHITECTURES or key is None):
            key = model_type        # a name nobody registered is reported as unsupported below
    if key is None:
        raise invalid_manifest("config.json names no architecture ('architectures' or 'model_type')")
    entry = _ARCHITECTURES.get(key)
    if entry is None:
        raise unsupported(f"unsupported model_type or architecture '{key}' "
                          f"(registered: {', '.join(registered_architectures())})")
    return entry


def spec_from_config(config: Mapping[str, Any]) -> Tuple[Architecture, Any, ModelSpec]:
    entry = resolve_architecture(config)
    typed = entry.config_type.from_dict(config)
    return entry, typed, entry.build_spec(typed)


_LOADED = False


def _load_builtin() -> None:
    global _LOADED
    if not _LOADED:
        _LOADED = True
        from .models import qwen3  # noqa: F401  (registers itself)
