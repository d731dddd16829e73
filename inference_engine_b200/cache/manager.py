"""The cache manager: pages of keys and values per request and cache group, plus slots for
per-request state of fixed size.  No torch; device memory is in ``cache/storage.py``.

A *cache group* is a set of layers with the same needs (same key/value heads and head size,
and either all positions or a window of the latest ones).  Each paged group has pages and a
page pool of its own and one block table per request: entry ``i`` is the page that holds
positions ``[i * page_size, (i + 1) * page_size)``, or ``-1`` once a window has passed it
and the page was given back.  Token ``p`` lives in flat slot
``table[p // page_size] * page_size + p % page_size`` (engine/runtime/block_manager.py:171-174).

Pages are taken when a request grows (``grow``), given back when it ends (``free``) or
when a window has passed them (``release_behind_window``), and used again first-in
first-out.  ``check_invariants`` verifies that no page is lost, held twice or both free
and held (engine/runtime/block_manager.py:176-191).
"""

from __future__ import annotations

from dataclasses import dataclass, field

from .pages import OutOfPages, PagePool, SlotPool


@dataclass(frozen=True)
class PagedGroupSpec:
    """Layers that keep keys and values per token."""

    num_layers: int
    num_kv_heads: int
    head_dim: int
    window: int | None = None  # None: every position stays; else the latest ``window`` do

    def bytes_per_page(self, page_size: int, dtype_bytes: int) -> int:
        return 2 * self.num_layers * self.num_kv_heads * self.head_dim * page_size * dtype_bytes


@dataclass(frozen=True)
class StateGroupSpec:
    """Layers that keep a 32-bit state of fixed ``shape`` per request."""

    num_layers: int
    shape: tuple[int, ...]


@dataclass
class _Request:
    tables: list[list[int]]  # one block table per paged group
    state_slot: int
    released: list[int] = field(default_factory=list)  # per group: pages given back in front


class CacheManager:
    def __init__(self, paged_groups: list[PagedGroupSpec], state_groups: list[StateGroupSpec],
                 num_pages: int | list[int], page_size: int, max_requests: int,
                 max_pages_per_request: int | None = None) -> None:
        if page_size < 1 or page_size & (page_size - 1):
            raise ValueError("page_size must be a power of two")
        self.paged_groups, self.state_groups = list(paged_groups), list(state_groups)
        self.page_size, self.max_requests = page_size, max_requests
        counts = [num_pages] * len(self.paged_groups) if isinstance(num_pages, int) else list(num_pages)
        if len(counts) != len(self.paged_groups):
            raise ValueError("num_pages needs one entry per paged cache group")
        self.pools = [PagePool(n) for n in counts]
        self._has_window = any(g.window is not None for g in self.paged_groups)
        self.slots = SlotPool(max_requests)
        self._requests: dict[object, _Request] = {}
        # A dense copy of the block tables, one row per state slot (the last row is the
        # padding row of fixed-size launches), kept in step with the lists: the step function
        # gathers the rows of a whole batch from it in one operation.  numpy is optional here.
        self.table_rows = None
        try:
            import numpy as np

            widths = [min(n, max_pages_per_request or n) for n in counts]
            self.table_rows = [np.full((max_requests + 1, w), -1, dtype=np.int32) for w in widths]
        except ImportError:  # pragma: no cover
            pass

    # --- sizes ------------------------------------------------------------------------------

    @property
    def capacity_tokens(self) -> int:
        """Tokens one request can hold at most (the smallest group decides)."""
        if not self.pools:
            return 2**62
        return min(p.num_pages for p in self.pools) * self.page_size

    @property
    def num_free_pages(self) -> list[int]:
        return [p.num_free for p in self.pools]

    def has_request(self, req_id) -> bool:
        return req_id in self._requests

    # --- requests ---------------------------------------------------------------------------

    def add_request(self, req_id) -> int:
        """Register a request (it holds no page yet) and give it a state slot."""
        if req_id in self._requests:
            raise ValueError(f"request {req_id!r} is already in the cache manager")
        slot = self.slots.allocate()
        self._requests[req_id] = _Request([[] for _ in self.paged_groups], slot,
                                          [0] * len(self.paged_groups))
        return slot

    def can_admit(self) -> bool:
        return self.slots.num_free > 0

    def state_slot(self, req_id) -> int:
        return self._requests[req_id].state_slot

    def table(self, group: int, req_id) -> list[int]:
        return self._requests[req_id].tables[group]

    def _first_needed_page(self, group: int, first_query_pos: int) -> int:
        window = self.paged_groups[group].window
        if window is None:
            return 0
        return max(first_query_pos - window + 1, 0) // self.page_size

    def pages_needed(self, req_id, num_computed: int, num_tokens: int) -> list[int]:
        """Extra pages per group so that positions up to ``num_tokens`` are held, given
        that the next query sits at ``num_computed``."""
        req = self._requests[req_id]
        last_page = -(-num_tokens // self.page_size)
        needed = []
        for g, table in enumerate(req.tables):
            first = self._first_needed_page(g, num_computed)
            n = 0
            for i in range(first, last_page):
                if i >= len(table) or table[i] < 0:
                    n += 1
            needed.append(n)
        return needed

    def missing_pages(self, req_id, num_computed: int, num_tokens: int) -> list[int] | None:
        """``pages_needed``, but None when no group needs a page: the usual case of a decoding
        request with room in its last page costs a few comparisons."""
        tables = self._requests[req_id].tables
        if not self._has_window:
            last_page = -(-num_tokens // self.page_size)
            if all(len(t) >= last_page for t in tables):
                return None
        need = self.pages_needed(req_id, num_computed, num_tokens)
        return need if any(need) else None

    def pages_for_new_request(self, num_tokens: int) -> list[int]:
        """Pages per group that a request not yet registered needs for its first
        ``num_tokens`` positions."""
        return [-(-num_tokens // self.page_size)] * len(self.paged_groups)

    def pages_held(self, req_id) -> list[int]:
        """Pages per group the request holds now (what it gives back when it is freed)."""
        return [sum(1 for page in t if page >= 0) for t in self._requests[req_id].tables]

    def can_grow(self, req_id, num_computed: int, num_tokens: int) -> bool:
        need = self.pages_needed(req_id, num_computed, num_tokens)
        return all(n <= pool.num_free for n, pool in zip(need, self.pools))

    def grow(self, req_id, num_computed: int, num_tokens: int) -> None:
        """Make room for positions ``[num_computed, num_tokens)`` (and, behind them, what a
        window still sees) in every group, or raise :class:`OutOfPages` and change nothing."""
        if not self.can_grow(req_id, num_computed, num_tokens):
            raise OutOfPages(f"request {req_id!r} needs "
                             f"{self.pages_needed(req_id, num_computed, num_tokens)} pages, "
                             f"free: {self.num_free_pages}")
        req = self._requests[req_id]
        last_page = -(-num_tokens // self.page_size)
        for g, table in enumerate(req.tables):
            first = self._first_needed_page(g, num_computed)
            while len(table) < last_page:
                table.append(-1)
            for i in range(first, last_page):
                if table[i] < 0:
                    table[i] = self.pools[g].allocate()
                    self._mirror(g, req.state_slot, i, table[i])

    def _mirror(self, group: int, slot: int, index: int, page: int) -> None:
        if self.table_rows is not None and index < self.table_rows[group].shape[1]:
            self.table_rows[group][slot, index] = page

    def try_grow(self, req_id, num_computed: int, num_tokens: int) -> bool:
        """``grow`` if there is room, in one pass; False (and nothing changed) otherwise.  The
        common case of a decoding request that still has room in its last page costs a few
        comparisons."""
        req = self._requests[req_id]
        last_page = -(-num_tokens // self.page_size)
        simple = True
        for g, table in enumerate(req.tables):
            if self.paged_groups[g].window is not None or len(table) < last_page:
                simple = False
                break
        if simple:
            return True
        if not self.can_grow(req_id, num_computed, num_tokens):
            return False
        self.grow(req_id, num_computed, num_tokens)
        return True

    def release_behind_window(self, req_id, num_computed: int) -> int:
        """Give back the pages no later query can see: those wholly before
        ``num_computed - window + 1`` in windowed groups.  Returns how many were freed."""
        if not self._has_window:
            return 0
        req = self._requests.get(req_id)
        if req is None:  # it ended meanwhile (a step launched before its last token was seen)
            return 0
        freed = 0
        for g, table in enumerate(req.tables):
            first = min(self._first_needed_page(g, num_computed), len(table))
            for i in range(req.released[g], first):
                if table[i] >= 0:
                    self.pools[g].free(table[i])
                    table[i] = -1
                    self._mirror(g, req.state_slot, i, -1)
                    freed += 1
            req.released[g] = max(req.released[g], first)
        return freed

    def release_pages(self, req_id) -> None:
        """Give back every page of a request but keep it registered (recompute preemption)."""
        req = self._requests[req_id]
        for g, table in enumerate(req.tables):
            for page in table:
                if page >= 0:
                    self.pools[g].free(page)
            if self.table_rows is not None:
                self.table_rows[g][req.state_slot, : len(table)] = -1
            table.clear()
            req.released[g] = 0

    def free(self, req_id) -> None:
        """The request ended: pages and state slot go back."""
        if req_id not in self._requests:
            return
        self.release_pages(req_id)
        self.slots.free(self._requests.pop(req_id).state_slot)

    def slot(self, group: int, req_id, position: int) -> int:
        page = self._requests[req_id].tables[group][position // self.page_size]
        if page < 0:
            raise ValueError(f"position {position} of {req_id!r} is no longer cached")
        return page * self.page_size + position % self.page_size

    # --- debugging --------------------------------------------------------------------------

    def check_invariants(self) -> None:
        for g, pool in enumerate(self.pools):
            owned: dict[int, int] = {}
            for req in self._requests.values():
                for page in req.tables[g]:
                    if page >= 0:
                        owned[page] = owned.get(page, 0) + 1
            free = pool.free_pages()
            assert len(set(free)) == len(free), f"group {g}: a page is twice in the free list"
            assert not set(free) & set(owned), f"group {g}: a page is both free and held"
            assert len(free) + len(owned) == pool.num_pages, f"group {g}: pages were lost"
            for page, n in owned.items():
                assert pool.refcount(page) == n, (
                    f"group {g}: page {page} has refcount {pool.refcount(page)} but {n} holders")
        slots = [r.state_slot for r in self._requests.values()]
        assert len(set(slots)) == len(slots), "a state slot is held twice"
        assert set(slots) == self.slots.used_slots(), "state slots and requests disagree"
        assert self.slots.num_free + len(slots) == self.slots.num_slots, "a state slot was lost"
