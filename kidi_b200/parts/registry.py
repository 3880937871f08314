"""Registries of parts by role and kind.

A part is registered under a role ("mixer", "feed_forward", "norm", "position",
"arrangement", "embedding", "head") and a kind (any string). `build_part` makes
one from a `PartSpec`. A test or a user can register a part of its own and name it
in a `ModelSpec` without touching this package.
"""
from __future__ import annotations

from typing import Callable, Dict

from ..errors import unsupported
from .spec import PartSpec

ROLES = ("mixer", "feed_forward", "norm", "position", "arrangement", "embedding", "head")

_PARTS: Dict[str, Dict[str, type]] = {role: {} for role in ROLES}


def register_part(role: str, kind: str) -> Callable[[type], type]:
    if role not in _PARTS:
        raise ValueError(f"unknown part role '{role}' (roles: {', '.join(ROLES)})")

    def decorate(cls: type) -> type:
        _PARTS[role][kind] = cls
        cls.role = role
        cls.kind = kind
        return cls

    return decorate


def part_class(role: str, kind: str) -> type:
    try:
        return _PARTS[role][kind]
    except KeyError:
        known = ", ".join(sorted(_PARTS.get(role, {}))) or "none"
        raise unsupported(f"no {role} part of kind '{kind}' is registered (registered: {known})") from None


def build_part(role: str, spec: PartSpec, env) -> "object":
    return part_class(role, spec.kind)(spec, env)


def registered_parts(role: str) -> Dict[str, type]:
    return dict(_PARTS[role])
