from __future__ import annotations

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_terminal_summary(terminalreporter):
    """The largest logit differences the comparisons with the plain implementation saw."""
    from tests import helpers

    for dtype, seen in sorted(helpers.ACHIEVED.items()):
        bounds = helpers.TOL[dtype]
        terminalreporter.write_line(
            f"logits vs plain implementation, {dtype}: " + ", ".join(
                f"{k} {v:.3g}" for k, v in sorted(seen.items())) + f"  (bounds: {bounds})")
