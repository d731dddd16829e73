"""Typed model configuration read from a Hugging Face style ``config.json``.

Every size and constant the engine uses comes from here: no part, kernel wrapper or
cache carries a model size of its own.  The Llama keys and their defaults follow the
reference's ``ModelConfig`` (engine/config.py:44-106) and ``RopeScaling``
(engine/config.py:16-41).  This module does not import torch.
"""

from __future__ import annotations

import json
import math
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """A ``config.json`` that the engine cannot use; the message names the key."""


def _require(raw: dict[str, Any], key: str, kind: type = int) -> Any:
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json is missing the required key {key!r}")
    try:
        return kind(raw[key])
    except (TypeError, ValueError) as exc:
        raise ConfigError(f"config.json key {key!r} = {raw[key]!r} is not a {kind.__name__}") from exc


def _as_id_tuple(value: Any) -> tuple[int, ...]:
    """``eos_token_id`` may be absent, one id or a list (engine/config.py:109-114)."""
    if value is None:
        return ()
    if isinstance(value, (list, tuple)):
        return tuple(int(v) for v in value)
    return (int(value),)


@dataclass(frozen=True)
class RopeScaling:
    """Llama 3 frequency scaling (engine/config.py:16-41): only ``llama3`` is accepted;
    the type is read from ``rope_type`` or the legacy ``type`` key."""

    rope_type: str
    factor: float
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> RopeScaling:
        rope_type = raw.get("rope_type") or raw.get("type")
        if rope_type != "llama3":
            raise ConfigError(f"unsupported rope_scaling type {rope_type!r}; only 'llama3' is")
        if "factor" not in raw:
            raise ConfigError("rope_scaling is missing the required key 'factor'")
        scaling = cls(
            rope_type=rope_type,
            factor=float(raw["factor"]),
            low_freq_factor=float(raw.get("low_freq_factor", 1.0)),
            high_freq_factor=float(raw.get("high_freq_factor", 4.0)),
            original_max_position_embeddings=int(raw.get("original_max_position_embeddings", 8192)),
        )
        if scaling.high_freq_factor == scaling.low_freq_factor:
            raise ConfigError("rope_scaling: high_freq_factor must differ from low_freq_factor")
        return scaling


@dataclass(frozen=True)
class LlamaConfig:
    """The Llama family's configuration; field for field the reference's ``ModelConfig``
    (engine/config.py:44-61) with the same defaults (engine/config.py:76-101)."""

    architecture: str
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: RopeScaling | None
    tie_word_embeddings: bool
    bos_token_id: int | None
    eos_token_ids: tuple[int, ...]
    torch_dtype: str

    @property
    def num_kv_groups(self) -> int:
        """Query heads that share one key/value head."""
        return self.num_attention_heads // self.num_key_value_heads

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> LlamaConfig:
        hidden = _require(raw, "hidden_size")
        n_heads = _require(raw, "num_attention_heads")
        n_kv = int(raw.get("num_key_value_heads") or n_heads)
        if n_heads < 1 or n_kv < 1:
            raise ConfigError("num_attention_heads and num_key_value_heads must be >= 1")
        if n_heads % n_kv:
            raise ConfigError(
                f"num_attention_heads ({n_heads}) not divisible by KV heads ({n_kv})"
            )
        head_dim = int(raw.get("head_dim") or hidden // n_heads)
        if head_dim < 2 or head_dim % 2:
            raise ConfigError(f"head_dim ({head_dim}) must be even: rotary pairs split it in half")
        scaling = raw.get("rope_scaling")
        cfg = cls(
            architecture=architecture_name(raw),
            vocab_size=_require(raw, "vocab_size"),
            hidden_size=hidden,
            intermediate_size=_require(raw, "intermediate_size"),
            num_hidden_layers=_require(raw, "num_hidden_layers"),
            num_attention_heads=n_heads,
            num_key_value_heads=n_kv,
            head_dim=head_dim,
            max_position_embeddings=int(raw.get("max_position_embeddings", 2048)),
            rms_norm_eps=float(raw.get("rms_norm_eps", 1e-5)),
            rope_theta=float(raw.get("rope_theta", 10000.0)),
            rope_scaling=RopeScaling.from_dict(scaling) if scaling else None,
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            bos_token_id=raw.get("bos_token_id"),
            eos_token_ids=_as_id_tuple(raw.get("eos_token_id")),
            torch_dtype=str(raw.get("torch_dtype", "bfloat16")),
        )
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                    "max_position_embeddings"):
            if getattr(cfg, key) < 1:
                raise ConfigError(f"config.json key {key!r} must be >= 1")
        if not cfg.rms_norm_eps > 0 or not math.isfinite(cfg.rms_norm_eps):
            raise ConfigError("rms_norm_eps must be a positive number")
        return cfg

    def to_dict(self) -> dict[str, Any]:
        """The ``config.json`` dictionary that parses back into this configuration."""
        raw = asdict(self)
        raw["architectures"] = [raw.pop("architecture")]
        eos = raw.pop("eos_token_ids")
        if eos:
            raw["eos_token_id"] = list(eos) if len(eos) > 1 else eos[0]
        if raw["rope_scaling"] is None:
            del raw["rope_scaling"]
        if raw["bos_token_id"] is None:
            del raw["bos_token_id"]
        return raw


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
    """``config.json``'s end-of-sequence ids followed by ``generation_config.json``'s,
    de-duplicated in order (engine/config.py:117-129)."""
    model_dir = Path(model_dir)
    ids = list(_as_id_tuple(read_config_dict(model_dir).get("eos_token_id")))
    gen_path = model_dir / "generation_config.json"
    if gen_path.exists():
        with open(gen_path, encoding="utf-8") as f:
            ids.extend(_as_id_tuple(json.load(f).get("eos_token_id")))
    return tuple(dict.fromkeys(ids))


# --- memory estimates (engine/config.py:135-162) -------------------------------------------


def estimate_param_count(cfg: LlamaConfig) -> int:
    """Exact number of parameters of a Llama model without biases."""
    h = cfg.hidden_size
    attn = h * cfg.q_size + 2 * h * cfg.kv_size + cfg.q_size * h
    mlp = 3 * h * cfg.intermediate_size
    per_layer = attn + mlp + 2 * h
    embed = cfg.vocab_size * h
    head = 0 if cfg.tie_word_embeddings else cfg.vocab_size * h
    return embed + cfg.num_hidden_layers * per_layer + h + head


def kv_bytes_per_token(cfg: LlamaConfig, dtype_bytes: int = 2) -> int:
    """Bytes of keys and values that one token adds over all layers."""
    return 2 * cfg.num_hidden_layers * cfg.kv_size * dtype_bytes


def max_kv_tokens(
    cfg: LlamaConfig,
    gpu_mem_gib: float,
    weight_bytes_per_param: float = 2.0,
    reserve_gib: float = 1.0,
) -> int:
    """Tokens of cache that fit beside the weights and a reserve for activations."""
    weights = estimate_param_count(cfg) * weight_bytes_per_param
    free = gpu_mem_gib * 2**30 - weights - reserve_gib * 2**30
    return max(0, int(free // kv_bytes_per_token(cfg)))
