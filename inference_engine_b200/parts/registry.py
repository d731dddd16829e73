"""Registries from a part's kind to its class, one per category.

A model description names parts by kind; :func:`build_part` looks the class up and calls
its ``from_spec(params, env, **context)``.  Registering a new kind (from anywhere, a test
included) is all it takes to make it available to model descriptions.
"""

from __future__ import annotations

from typing import Any

from ..config.spec import PartSpec
from .base import BuildEnv

CATEGORIES = ("norm", "position", "mixer", "feed_forward", "block", "embedding", "head")
_REGISTRY: dict[str, dict[str, type]] = {c: {} for c in CATEGORIES}


def register_part(category: str, kind: str, cls: type | None = None, replace: bool = False):
    """``register_part("mixer", "my_mixer", MyMixer)`` or as a class decorator."""
    if category not in _REGISTRY:
        raise ValueError(f"unknown part category {category!r}; one of {CATEGORIES}")

    def _register(c: type) -> type:
        if kind in _REGISTRY[category] and not replace:
            raise ValueError(f"{category} kind {kind!r} is already registered")
        _REGISTRY[category][kind] = c
        return c

    return _register(cls) if cls is not None else _register


def registered_kinds(category: str) -> list[str]:
    return sorted(_REGISTRY[category])


def build_part(category: str, spec: PartSpec, env: BuildEnv, **context: Any):
    try:
        cls = _REGISTRY[category][spec.kind]
    except KeyError:
        raise ValueError(
            f"no {category} of kind {spec.kind!r}; registered: {registered_kinds(category)}"
        ) from None
    return cls.from_spec(dict(spec.params), env, **context)
