"""One registry from an architecture's name to its configuration class and model builder.

``config.json`` names the architecture (``architectures[0]``, else ``model_type``); the
registry gives the typed configuration class that parses the file and the function that
turns that configuration into a :class:`~inference_engine_b200.config.spec.ModelSpec`.
The reference has only a set of supported names (engine/config.py:13) and hard-codes the
model class in its loader (engine/model/loader.py:60,72).
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

from .model_config import ConfigError, Footprint, architecture_name, read_config_dict
from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type  # has ``from_dict(raw) -> config``
    build_spec: Callable[[Any], ModelSpec]
    describe: Callable[[Any], list[str]] | None = None  # the lines `engine info` prints about the shape
    footprint: Callable[[Any], Footprint] | None = None  # parameters and cache per token, without building the model


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(
    name: str,
    config_class: type,
    build_spec: Callable[[Any], ModelSpec],
    describe: Callable[[Any], list[str]] | None = None,
    footprint: Callable[[Any], Footprint] | None = None,
    replace: bool = False,
) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, config_class, build_spec, describe, footprint)


def _load_builtin() -> None:
    """The package's own architectures register themselves when their module is imported."""
    from .. import architectures  # noqa: F401


def supported_architectures() -> list[str]:
    _load_builtin()
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    _load_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unsupported architecture {name!r}; supported: {supported_architectures()}"
        ) from None


def config_from_dict(raw: dict[str, Any]) -> Any:
    """Parse a ``config.json`` dictionary with the class its architecture registered."""
    return get_architecture(architecture_name(raw)).config_class.from_dict(raw)


def load_config(model_dir: str | Path) -> Any:
    return config_from_dict(read_config_dict(model_dir))


def build_model_spec(config: Any) -> ModelSpec:
    spec = get_architecture(config.architecture).build_spec(config)
    spec.validate()
    return spec
