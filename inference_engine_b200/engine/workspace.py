"""Named device buffers that live across steps.

Every intermediate of a step is a view of a buffer that was allocated once for the most
tokens a step may hold, so steady-state steps allocate nothing and a captured launch
sequence keeps reading and writing the same addresses.  ``version`` changes whenever a
buffer had to be replaced by a larger one; whoever captured addresses must capture again.
"""

from __future__ import annotations


class Workspace:
    def __init__(self, device, min_rows: int = 1) -> None:
        self.device, self.min_rows = device, max(int(min_rows), 1)
        self._buffers: dict[str, object] = {}
        self._views: dict[tuple, tuple] = {}  # last view handed out per buffer
        self.version = 0

    def buffer(self, name: str, rows: int, cols: int, dtype, rows_cap: int | None = 0):
        """A ``[rows, cols]`` view named ``name``.  Capacity is at least ``min_rows`` rows
        (``rows_cap=None``: exactly what is asked for, for buffers that are rarely large)."""
        key = (name, dtype)  # the same name may be wanted in two precisions by different paths
        hit = self._views.get(key)
        if hit is not None and hit[0] == rows and hit[1] == cols:
            return hit[2]  # the same view as last time: a step asks for every buffer once per layer
        import torch

        need = rows * cols
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < need:
            cap_rows = rows if rows_cap is None else max(rows, self.min_rows, rows_cap)
            buf = torch.empty(max(cap_rows * cols, 1), dtype=dtype, device=self.device)
            if key in self._buffers:
                self.version += 1
            self._buffers[key] = buf
        view = buf[:need].view(rows, cols)
        self._views[key] = (rows, cols, view)
        return view

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())
