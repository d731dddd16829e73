"""Bookkeeping of fixed-size cache pages and of per-request state slots.  No torch.

The free list is first-in first-out, as the reference's block allocator
(engine/runtime/block_manager.py:33,44-53,66-74): a page given back is the last to be
handed out again.  Reference counts are kept so that sharing can be added; today every page
has at most one owner.
"""

from __future__ import annotations

from collections import deque


class OutOfPages(RuntimeError):
    """No free page (or slot).  The scheduler checks ``can_grow`` first, so this is a bug
    or a direct caller asking for too much."""


class PagePool:
    def __init__(self, num_pages: int) -> None:
        if num_pages < 1:
            raise ValueError("num_pages must be >= 1")
        self.num_pages = num_pages
        self._free: deque[int] = deque(range(num_pages))
        self._refs = [0] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages("no free cache page")
        page = self._free.popleft()
        self._refs[page] = 1
        return page

    def incref(self, page: int) -> None:
        if self._refs[page] < 1:
            raise ValueError(f"page {page} is free; it cannot be shared")
        self._refs[page] += 1

    def free(self, page: int) -> None:
        if not 0 <= page < self.num_pages:
            raise ValueError(f"page {page} does not exist")
        if self._refs[page] < 1:
            raise ValueError(f"double free of page {page}")
        self._refs[page] -= 1
        if self._refs[page] == 0:
            self._free.append(page)

    def refcount(self, page: int) -> int:
        return self._refs[page]

    def free_pages(self) -> list[int]:
        return list(self._free)


class SlotPool:
    """Slots for per-request state of fixed size: one slot index per live request, handed
    out at admission and given back when the request ends."""

    def __init__(self, num_slots: int) -> None:
        if num_slots < 1:
            raise ValueError("num_slots must be >= 1")
        self.num_slots = num_slots
        self._free: deque[int] = deque(range(num_slots))
        self._used: set[int] = set()

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages("no free state slot")
        slot = self._free.popleft()
        self._used.add(slot)
        return slot

    def free(self, slot: int) -> None:
        if slot not in self._used:
            raise ValueError(f"double free of state slot {slot}")
        self._used.remove(slot)
        self._free.append(slot)

    def used_slots(self) -> set[int]:
        return set(self._used)
