"""Weights from safetensors files, by tensor name.

File discovery follows engine/model/loader.py:18-29: the sharded index's files if there is
one, else ``model.safetensors``.  Tensors keep the precision they are stored in: bfloat16
stays bfloat16, 32-bit floats stay 32-bit, half floats become bfloat16, integer tables
become int32.  Before anything is read, the names and shapes in the files are compared with
what the model declares, and every difference is reported in one error.
"""

from __future__ import annotations

import json
import logging
from pathlib import Path
from typing import Any

log = logging.getLogger(__name__)


class WeightError(RuntimeError):
    """The checkpoint does not fit the model.  ``missing``, ``unexpected`` and
    ``wrong_shape`` hold the tensor names; the message lists all three."""

    def __init__(self, missing: list[str], unexpected: list[str],
                 wrong_shape: list[tuple[str, tuple, tuple]], where: str = "") -> None:
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong_shape
        lines = [f"checkpoint {where} does not fit the model:".replace("  ", " ")]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shapes ({len(wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in wrong_shape))
        super().__init__("\n".join(lines))


def find_safetensors_files(model_dir: str | Path) -> list[Path]:
    """The checkpoint's files: the shards that ``model.safetensors.index.json`` maps tensors to
    (each once, by name), else the single ``model.safetensors``
    (engine/model/loader.py:18-29)."""
    folder = Path(model_dir)
    index_file = folder / "model.safetensors.index.json"
    if not index_file.exists():
        whole = folder / "model.safetensors"
        if whole.exists():
            return [whole]
        raise FileNotFoundError(f"no safetensors weights in {folder}")
    shard_of = json.loads(index_file.read_text(encoding="utf-8"))["weight_map"]
    return [folder / shard for shard in sorted(set(shard_of.values()))]


def check_names_and_shapes(found: dict[str, tuple[int, ...]], expected: dict[str, Any],
                           where: str = "") -> None:
    """``found``: name -> shape in the files; ``expected``: name -> WeightDecl."""
    missing = sorted(n for n in expected if n not in found)
    unexpected = sorted(n for n in found if n not in expected)
    wrong = sorted(
        (n, tuple(found[n]), tuple(expected[n].shape))
        for n in expected if n in found and tuple(found[n]) != tuple(expected[n].shape)
    )
    if missing or unexpected or wrong:
        raise WeightError(missing, unexpected, wrong, where)


def stored_dtype(dtype):
    """The dtype a stored tensor is kept in."""
    import torch

    if dtype in (torch.bfloat16, torch.float32):
        return dtype
    if dtype == torch.float16:
        return torch.bfloat16
    if dtype == torch.float64:
        return torch.float32
    if not dtype.is_floating_point:
        return torch.int32
    raise WeightError([], [], [], f"(unsupported stored dtype {dtype})")


def load_weights(model_dir: str | Path, expected: dict[str, Any], device) -> dict[str, Any]:
    """Read the tensors ``expected`` names from ``model_dir`` onto ``device``.

    Shards are opened once to compare names and shapes (nothing is copied for that), then
    read tensor by tensor so the host never holds more than one tensor beside the file map.
    """
    from safetensors import safe_open

    files = find_safetensors_files(model_dir)
    found: dict[str, tuple[int, ...]] = {}
    owner: dict[str, Path] = {}
    for path in files:
        with safe_open(str(path), framework="pt", device="cpu") as f:
            for name in f.keys():
                found[name] = tuple(f.get_slice(name).get_shape())
                owner[name] = path
    check_names_and_shapes(found, expected, where=f"in {model_dir}")
    tensors: dict[str, Any] = {}
    total = 0
    for path in files:
        with safe_open(str(path), framework="pt", device="cpu") as f:
            for name in f.keys():
                if owner[name] != path:
                    continue
                t = f.get_tensor(name)
                t = t.to(stored_dtype(t.dtype)).to(device)
                total += t.numel()
                tensors[name] = t
    log.info("loaded %.2f B parameters from %s", total / 1e9, model_dir)
    return tensors
