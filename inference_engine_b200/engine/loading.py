"""From a model folder (or a configuration and a seed) to a loaded :class:`Model`.

Steps as in engine/model/loader.py:32-120: read ``config.json``, build the model without
weights, read the tensors shard by shard, hand them over, tie the head.  The model class is
chosen by ``config.json`` through the architecture registry.
"""

from __future__ import annotations

import logging
from pathlib import Path
from typing import Any

from .. import architectures  # noqa: F401 (registers the built-in architectures)
from ..config.registry import build_model_spec, config_from_dict, load_config
from ..weights.loader import check_names_and_shapes, load_weights
from ..weights.random_weights import random_tensors
from .model import Model

log = logging.getLogger(__name__)


def load_model(model_dir: str | Path, dtype: str = "bfloat16", device="cuda",
               max_positions: int | None = None) -> tuple[Model, Any]:
    """Returns ``(model, config)``."""
    cfg = load_config(model_dir)
    spec = build_model_spec(cfg)
    model = Model(spec, dtype, max_positions or spec.max_position_embeddings, device)
    model.load(load_weights(model_dir, model.declared_weights(), device))
    return model, cfg


def random_model(config: dict[str, Any] | Any, seed: int = 0, dtype: str = "bfloat16",
                 device="cuda", max_positions: int | None = None, std: float = 0.02,
                 stored_dtype=None) -> tuple[Model, Any]:
    """A model with seeded random weights drawn straight on ``device`` (no folder)."""
    import torch

    cfg = config_from_dict(config) if isinstance(config, dict) else config
    spec = build_model_spec(cfg)
    model = Model(spec, dtype, max_positions or spec.max_position_embeddings, device)
    tensors = random_tensors(model.declared_weights(), seed, std,
                             stored_dtype or torch.bfloat16, device)
    model.load(tensors)
    return model, cfg


def model_from_tensors(config: dict[str, Any], tensors: dict[str, Any], dtype: str, device,
                       max_positions: int | None = None) -> tuple[Model, Any]:
    cfg = config_from_dict(config)
    spec = build_model_spec(cfg)
    model = Model(spec, dtype, max_positions or spec.max_position_embeddings, device)
    expected = model.declared_weights()
    check_names_and_shapes({n: tuple(t.shape) for n, t in tensors.items()}, expected)
    model.load({n: t.to(device) for n, t in tensors.items()})
    return model, cfg
