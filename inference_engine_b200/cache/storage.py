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
