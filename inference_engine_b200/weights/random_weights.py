"""Seeded random weights: for a model in memory, or written out as a model folder.

Every tensor is drawn from its own generator seeded by ``(seed, tensor name)``, so a
tensor's values do not depend on which other tensors exist, on the order of generation or
on the dtype asked for: matrices are N(0, std), norm weights 1 + N(0, std).  Values are
drawn in 32-bit and rounded to the stored dtype.  The reference has no such mode (its
tests use the default ``nn.Module`` initialisation under one global seed,
tests/test_engine.py:32-33).
"""

from __future__ import annotations

import json
import zlib
from pathlib import Path
from typing import Any


def _tensor_seed(seed: int, name: str) -> int:
    return (int(seed) * 0x9E3779B1 + zlib.crc32(name.encode("utf-8"))) % (2**63 - 1)


def random_tensor(name: str, decl: Any, seed: int, std: float, dtype, device="cpu"):
    import torch

    gen = torch.Generator(device=device).manual_seed(_tensor_seed(seed, name))
    if decl.init == "zeros":
        t = torch.zeros(decl.shape, dtype=torch.float32, device=device)
    elif decl.init == "ones":
        t = torch.ones(decl.shape, dtype=torch.float32, device=device)
    else:
        t = torch.randn(decl.shape, generator=gen, dtype=torch.float32, device=device) * std
        if decl.init == "ones_plus_normal":
            t += 1.0
    if decl.role == "int_table":
        return t.to(torch.int32)
    return t.to(dtype)


def random_tensors(expected: dict[str, Any], seed: int, std: float = 0.02, dtype=None,
                   device="cpu") -> dict[str, Any]:
    import torch

    dtype = dtype or torch.bfloat16
    return {n: random_tensor(n, d, seed, std, dtype, device) for n, d in expected.items()}


def write_random_model(config: dict[str, Any], out_dir: str | Path, seed: int = 0,
                       std: float = 0.02, dtype: str = "bfloat16") -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a ``config.json``
    dictionary of a registered architecture) with seeded random weights."""
    import torch
    from safetensors.torch import save_file

    from ..config.registry import build_model_spec, config_from_dict
    from ..engine.model import declared_weights

    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    cfg = config_from_dict(config)
    expected = declared_weights(build_model_spec(cfg))
    torch_dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    tensors = random_tensors(expected, seed, std, torch_dtype)
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(out_dir / "model.safetensors"))
    raw = dict(config)
    raw["torch_dtype"] = dtype
    with open(out_dir / "config.json", "w", encoding="utf-8") as f:
        json.dump(raw, f, indent=2)
    return out_dir
