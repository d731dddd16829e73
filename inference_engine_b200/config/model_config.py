"""What every architecture's configuration shares: reading ``config.json``, the error type,
helpers for typed keys, stop ids, and the memory footprint an architecture reports.

The typed configuration itself belongs to the architecture (``architectures/llama.py`` has
Llama's); this module knows no model.  It does not import torch.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """A ``config.json`` that the engine cannot use; the message names the key."""


def require(raw: dict[str, Any], key: str, kind: type = int) -> Any:
    """``raw[key]`` as ``kind``; a missing key or a value of the wrong kind is a ConfigError."""
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json is missing the required key {key!r}")
    try:
        return kind(raw[key])
    except (TypeError, ValueError) as exc:
        raise ConfigError(f"config.json key {key!r} = {raw[key]!r} is not a {kind.__name__}") from exc


def id_tuple(value: Any) -> tuple[int, ...]:
    """Token ids given as nothing, one number or a list of numbers."""
    if isinstance(value, (list, tuple)):
        return tuple(map(int, value))
    return () if value is None else (int(value),)


def architecture_name(raw: dict[str, Any]) -> str:
    """``architectures[0]``, else ``model_type`` (engine/config.py:70-71)."""
    archs = raw.get("architectures") or []
    return str(archs[0]) if archs else str(raw.get("model_type", "unknown"))


def read_config_dict(model_dir: str | Path) -> dict[str, Any]:
    path = Path(model_dir) / "config.json"
    if not path.exists():
        raise FileNotFoundError(f"no config.json in {model_dir}")
    with open(path, encoding="utf-8") as f:
        return json.load(f)


def load_stop_token_ids(model_dir: str | Path) -> tuple[int, ...]:
    """The end-of-sequence ids a model folder names: those of ``config.json``, then those of
    ``generation_config.json`` if there is one, each id once (engine/config.py:117-129)."""
    folder = Path(model_dir)
    found: dict[int, None] = dict.fromkeys(id_tuple(read_config_dict(folder).get("eos_token_id")))
    generation = folder / "generation_config.json"
    if generation.exists():
        found.update(dict.fromkeys(id_tuple(json.loads(generation.read_text("utf-8")).get("eos_token_id"))))
    return tuple(found)


@dataclass(frozen=True)
class Footprint:
    """What a model costs in device memory, as its architecture reports it: parameters, cache
    values one token adds over all layers (keys and values), and values of fixed-size state
    one live request holds."""

    parameters: int
    cache_values_per_token: int
    state_values_per_request: int = 0

    def cache_bytes_per_token(self, dtype_bytes: int = 2) -> int:
        return self.cache_values_per_token * dtype_bytes

    def cache_tokens_that_fit(self, gpu_mem_gib: float, weight_bytes_per_param: float = 2.0,
                              reserve_gib: float = 1.0, cache_dtype_bytes: int = 2) -> int:
        """Tokens of cache beside the weights and a reserve (activations, CUDA context) on a
        device of ``gpu_mem_gib`` (engine/config.py:149-162)."""
        left = (gpu_mem_gib - reserve_gib) * 2**30 - self.parameters * weight_bytes_per_param
        per_token = max(self.cache_bytes_per_token(cache_dtype_bytes), 1)
        return int(left // per_token) if left > 0 else 0
