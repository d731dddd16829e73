"""Llama: its typed configuration, and how that becomes a model description.

Configuration keys and defaults follow the reference's ``ModelConfig`` and ``RopeScaling``
(engine/config.py:16-106).  Tensor names are Hugging Face's (engine/model/llama.py:3-8).
Every layer is a pre-norm residual block of grouped-query attention with rotary position
encoding and a gated feed-forward; layers run once each, in order; the head is tied to the
embedding table when ``tie_word_embeddings`` is set (the reference ties in its loader,
engine/model/loader.py:91-92,100-101).  No torch import here.
"""

from __future__ import annotations

import math
from dataclasses import asdict, dataclass
from typing import Any

from ..config.model_config import ConfigError, Footprint, architecture_name, id_tuple, require
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


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
    """The Llama family's configuration: the reference's ``ModelConfig`` fields
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
        hidden = require(raw, "hidden_size")
        n_heads = require(raw, "num_attention_heads")
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
            vocab_size=require(raw, "vocab_size"),
            hidden_size=hidden,
            intermediate_size=require(raw, "intermediate_size"),
            num_hidden_layers=require(raw, "num_hidden_layers"),
            num_attention_heads=n_heads,
            num_key_value_heads=n_kv,
            head_dim=head_dim,
            max_position_embeddings=int(raw.get("max_position_embeddings", 2048)),
            rms_norm_eps=float(raw.get("rms_norm_eps", 1e-5)),
            rope_theta=float(raw.get("rope_theta", 10000.0)),
            rope_scaling=RopeScaling.from_dict(scaling) if scaling else None,
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            bos_token_id=raw.get("bos_token_id"),
            eos_token_ids=id_tuple(raw.get("eos_token_id")),
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


def llama_footprint(cfg: LlamaConfig) -> Footprint:
    """Parameters counted matrix by matrix (no biases), and the keys and values a token adds
    (the reference's estimates, engine/config.py:135-146)."""
    h, layers = cfg.hidden_size, cfg.num_hidden_layers
    matrices = {
        "q_proj": cfg.q_size * h, "k_proj": cfg.kv_size * h, "v_proj": cfg.kv_size * h,
        "o_proj": h * cfg.q_size, "gate_proj": cfg.intermediate_size * h,
        "up_proj": cfg.intermediate_size * h, "down_proj": h * cfg.intermediate_size,
        "input_layernorm": h, "post_attention_layernorm": h,
    }
    tables = cfg.vocab_size * h * (1 if cfg.tie_word_embeddings else 2)
    return Footprint(parameters=tables + layers * sum(matrices.values()) + h,
                     cache_values_per_token=2 * layers * cfg.kv_size)


def llama_spec(cfg: LlamaConfig) -> ModelSpec:
    scaling = None
    if cfg.rope_scaling is not None:
        scaling = asdict(cfg.rope_scaling)
    positions = {
        "rotary": PartSpec("rotary", {
            "rotary_dim": cfg.head_dim, "theta": cfg.rope_theta, "scaling": scaling,
        })
    }
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        layers.append(LayerSpec(
            prefix=p,
            block=PartSpec("prenorm_residual"),
            mixer=PartSpec("paged_attention", {
                "q_proj": f"{p}.self_attn.q_proj.weight",
                "k_proj": f"{p}.self_attn.k_proj.weight",
                "v_proj": f"{p}.self_attn.v_proj.weight",
                "o_proj": f"{p}.self_attn.o_proj.weight",
                "num_heads": cfg.num_attention_heads,
                "num_kv_heads": cfg.num_key_value_heads,
                "head_dim": cfg.head_dim,
                "position": "rotary",
                "window": None,
            }),
            feed_forward=PartSpec("swiglu", {
                "gate_proj": f"{p}.mlp.gate_proj.weight",
                "up_proj": f"{p}.mlp.up_proj.weight",
                "down_proj": f"{p}.mlp.down_proj.weight",
                "intermediate_size": cfg.intermediate_size,
            }),
            norms={
                "pre_mixer": PartSpec("rms", {
                    "weight": f"{p}.input_layernorm.weight", "eps": cfg.rms_norm_eps}),
                "pre_feed_forward": PartSpec("rms", {
                    "weight": f"{p}.post_attention_layernorm.weight", "eps": cfg.rms_norm_eps}),
            },
        ))
    return ModelSpec(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        max_position_embeddings=cfg.max_position_embeddings,
        embedding=PartSpec("token", {
            "weight": "model.embed_tokens.weight", "vocab_size": cfg.vocab_size}),
        positions=positions,
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rms", {"weight": "model.norm.weight", "eps": cfg.rms_norm_eps}),
        head=PartSpec("linear", {
            "weight": None if cfg.tie_word_embeddings else "lm_head.weight",
            "vocab_size": cfg.vocab_size}),
        eos_token_ids=cfg.eos_token_ids,
        bos_token_id=cfg.bos_token_id,
    )


def describe_llama(cfg: LlamaConfig) -> list[str]:
    """The lines ``engine info`` prints about the shape (engine/cli.py:24-33)."""
    return [
        f"architecture        {cfg.architecture}",
        f"layers / hidden     {cfg.num_hidden_layers} / {cfg.hidden_size}",
        f"heads (q / kv)      {cfg.num_attention_heads} / {cfg.num_key_value_heads}"
        f"  (GQA groups: {cfg.num_kv_groups}, head dim {cfg.head_dim})",
        f"parameters          {llama_footprint(cfg).parameters / 1e9:.2f} B",
        f"KV cache per token  {llama_footprint(cfg).cache_bytes_per_token(2) / 1024:.0f} KiB (bf16)",
    ]


register_architecture("LlamaForCausalLM", LlamaConfig, llama_spec, describe_llama, llama_footprint)
