"""Device memory behind the cache manager's pages and state slots.

Per paged group two tensors ``k`` and ``v`` of shape
``[layers_in_group, num_pages + 1, kv_heads, page_size, head_dim]``: a page of one head is
contiguous (``page_size * head_dim`` elements), so a kernel reads a head's keys of a page
as one block.  The extra last page is scratch: padded rows of a fixed-size launch point
there.  Per state group one 32-bit tensor ``[layers_in_group, max_requests + 1, *shape]``.
The reference keeps ``[layers, slots, kv_heads, head_dim]`` (engine/runtime/paged_cache.py:31-35).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .manager import CacheManager


@dataclass
class PagedStorage:
    k: Any
    v: Any
    page_size: int
    num_pages: int  # without the scratch page
    window: int | None

    @property
    def scratch_page(self) -> int:
        return self.num_pages


HEADROOM_BYTES = 512 * 2**20  # left free beside the cache for activations and libraries' workspaces


def pages_that_fit(paged_groups, page_size: int, dtype_bytes: int, device, utilization: float) -> int:
    """How many pages per cache group the device has room for.  The engine may fill the
    fraction ``utilization`` of the device; what is taken already (weights, other processes)
    counts against that, and ``HEADROOM_BYTES`` stay free.  Every group gets the same number
    of pages, so a page costs the sum over the groups (the reference sizes its one pool the
    same way, engine/runtime/engine.py:130-140)."""
    import torch

    if not str(device).startswith("cuda"):
        raise ValueError("pass num_blocks explicitly when not running on CUDA")
    free_now, capacity = torch.cuda.mem_get_info(device)
    taken = capacity - free_now
    room = utilization * capacity - taken - HEADROOM_BYTES
    page_bytes = sum(g.bytes_per_page(page_size, dtype_bytes) for g in paged_groups)
    pages = int(room // page_bytes) if page_bytes else 1
    if pages < 1:
        raise RuntimeError(f"no GPU memory left for the KV cache ({free_now / 2**30:.1f} GiB free of "
                           f"{capacity / 2**30:.1f}, gpu_memory_utilization {utilization})")
    return pages


class CacheStorage:
    def __init__(self, manager: CacheManager, dtype, device) -> None:
        import torch

        self.paged: list[PagedStorage] = []
        for spec, pool in zip(manager.paged_groups, manager.pools):
            shape = (spec.num_layers, pool.num_pages + 1, spec.num_kv_heads,
                     manager.page_size, spec.head_dim)
            self.paged.append(PagedStorage(
                torch.zeros(shape, dtype=dtype, device=device),
                torch.zeros(shape, dtype=dtype, device=device),
                manager.page_size, pool.num_pages, spec.window))
        self.state = [
            torch.zeros((spec.num_layers, manager.max_requests + 1, *spec.shape),
                        dtype=torch.float32, device=device)
            for spec in manager.state_groups
        ]

    def bytes(self) -> int:
        total = sum(p.k.numel() * p.k.element_size() * 2 for p in self.paged)
        return total + sum(s.numel() * 4 for s in self.state)
