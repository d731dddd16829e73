"""The step function.

``ModelRunner.step(entries)`` runs exactly the tokens it is given, as one batch, against the
cache that earlier steps left, writes their keys and values into the requests' pages, and
returns 32-bit logits at the wanted places (none, some or all).  The reference's counterpart
is the device half of ``LLMEngine.step`` (engine/runtime/engine.py:186-227 with
engine/runtime/paged_cache.py:79-229); it returns the last row of every sequence, this
returns the rows that are asked for.

Pages must have been taken from the cache manager before the step (``grow``); the runner
only reads the block tables.
"""

from __future__ import annotations

import itertools
from typing import Any

from ..cache.manager import CacheManager
from ..cache.storage import CacheStorage
from .batch import PagedGroupView, StateGroupView, StepContext, StepEntry
from .model import Model
from .workspace import Workspace


def _align4(n: int) -> int:
    return (n + 3) & ~3


class ModelRunner:
    def __init__(self, model: Model, cache: CacheManager, storage: CacheStorage, ops,
                 device, max_tokens_per_step: int, max_seqs_per_step: int) -> None:
        import torch

        self.model, self.cache, self.storage, self.ops, self.device = model, cache, storage, ops, device
        self.max_tokens, self.max_seqs = int(max_tokens_per_step), int(max_seqs_per_step)
        self.ws = Workspace(device, min_rows=self.max_tokens)
        self.page_size = cache.page_size
        self._torch = torch
        self._staging_host = None
        self._staging_dev = None
        self.last_h2d_bytes = 0
        self._ensure_staging(self._staging_ints(self.max_tokens, self.max_seqs, self.max_seqs, 8))

    def contexts_are_ragged(self, ctx_lens) -> tuple[int, ...]:
        """A hint for the attention's launch, one answer per paged cache group: 1 if these
        requests' contexts (what a group's window leaves of them) differ so much in length that
        work dealt request by request would leave most of the GPU waiting for the longest one,
        2 or 3 if they are so many and so alike that blocks of as many warps pay, else 0.
        The kernels' side decides (it knows how many requests the device takes at once and the
        group's number of key/value heads and head size); without such kernels the answer is 0."""
        decide = getattr(self.ops, "decode_dealing", None)
        groups = self.cache.paged_groups
        if decide is None or len(ctx_lens) < 2:
            return (0,) * len(groups)
        answers = []
        for g in groups:
            seen = ctx_lens if g.window is None else [min(c, g.window) for c in ctx_lens]
            answers.append(int(decide(seen, g.num_kv_heads, getattr(g, "head_dim", None))))
        return tuple(answers)

    # --- staging ----------------------------------------------------------------------------

    def _staging_ints(self, n: int, b: int, r: int, width: int) -> int:
        groups = len(self.cache.paged_groups)
        per_group = _align4(n) + _align4(b * width)
        return (3 * _align4(n) + _align4(b + 1) + 3 * _align4(b) + _align4(r)
                + groups * per_group + 16)

    RING = 4  # pinned host buffers in rotation: a step may be packed while earlier copies wait

    def _ensure_staging(self, ints: int) -> None:
        torch = self._torch
        if self._staging_host is not None and self._staging_host[0].numel() >= ints:
            return
        cuda = self.device is not None and str(self.device).startswith("cuda")
        if cuda and self._staging_host is not None:
            torch.cuda.synchronize()  # copies from the old buffers may still be queued
        self._staging_host = [torch.empty(ints, dtype=torch.int32, pin_memory=cuda)
                              for _ in range(self.RING)]
        self._staging_events = [torch.cuda.Event() if cuda else None for _ in range(self.RING)]
        self._staging_used = [False] * self.RING
        self._staging_turn = 0
        self._staging_dev = torch.empty(ints, dtype=torch.int32, device=self.device)
        self.ws.version += 1

    def _next_host_buffer(self):
        """The next pinned buffer of the ring, once the copy that last read it has run."""
        i = self._staging_turn = (self._staging_turn + 1) % self.RING
        if self._staging_used[i] and self._staging_events[i] is not None:
            self._staging_events[i].synchronize()
        return i, self._staging_host[i].numpy()

    # --- one step ---------------------------------------------------------------------------

    def build_context(self, entries: list[StepEntry], pad_to_seqs: int | None = None,
                      table_width: int | None = None, views: bool = True,
                      pad_to_tokens: int | None = None, pad_to_rows: int | None = None):
        """Pack the step's index data, copy it to the device and return the context and the
        device vector of wanted rows.  ``pad_to_seqs``/``table_width`` give a launch of fixed
        size: missing sequences become single tokens that read and write the scratch page.
        With ``pad_to_tokens`` (and ``pad_to_rows`` wanted rows) the number of tokens is fixed
        too: the tokens beyond the step's own belong to no sequence (their keys and values go to
        the scratch page), and the sequences beyond the step's own hold no tokens."""
        import numpy as np

        torch = self._torch
        ps = self.page_size
        q_lens = [len(e.tokens) for e in entries]
        if any(n < 1 for n in q_lens):
            raise ValueError("every entry of a step needs at least one token")
        if max(q_lens) == 1 and self.cache.table_rows is not None and pad_to_tokens is None:
            return self._build_decode_context(entries, pad_to_seqs, table_width, views)
        real_b = len(entries)
        b = max(pad_to_seqs or 0, real_b)
        pad = b - real_b
        n = sum(q_lens) + pad
        rows = sum(len(e.want) for e in entries) + pad
        pad_tokens = 0
        if pad_to_tokens is not None:
            pad_tokens = pad_to_tokens - sum(q_lens)
            pad = 0  # (no single-token sequences: see below)
            n = pad_to_tokens
            rows = max(pad_to_rows or 0, sum(len(e.want) for e in entries), 1)
            if pad_tokens < 0 or b < real_b + (1 if pad_tokens else 0):
                raise ValueError(f"{sum(q_lens)} tokens of {real_b} sequences do not fit a launch of "
                                 f"{pad_to_tokens} tokens and {b} sequences")
        dense = self.cache.table_rows  # the block tables as arrays, a row per state slot (if numpy is there)
        if dense is not None:
            tables = [None] * len(self.cache.paged_groups)
            last_page = max((e.start + ql - 1) // ps for e, ql in zip(entries, q_lens))
            width = max(table_width or 1, last_page + 1)
        else:
            tables = [[self.cache.table(g, e.req_id) for e in entries]
                      for g in range(len(self.cache.paged_groups))]
            width = max([table_width or 1] + [len(t) for g in tables for t in g])
        self._ensure_staging(self._staging_ints(n, b, rows, width))
        turn, buf = self._next_host_buffer()
        off = 0

        def take(count: int):
            nonlocal off
            view = (off, count)
            off += _align4(count)
            return view

        v_tok, v_pos, v_seq = take(n), take(n), take(n)
        v_cu, v_ctx, v_state, v_rows = take(b + 1), take(b), take(b), take(rows)
        v_order = take(b)
        v_slots = [take(n) for _ in tables]
        v_tables = [take(b * width) for _ in tables]

        q_starts, start_positions, logit_rows, cursor = [], [], [], 0
        if dense is not None:
            # without a Python loop over what the entries hold (a step of thirty decoding requests
            # and a prompt is packed in a tenth of the time): per-token arrays from per-sequence ones
            q_arr = np.asarray(q_lens, dtype=np.int64)
            starts = np.fromiter((e.start for e in entries), dtype=np.int64, count=real_b)
            cu = np.concatenate(([0], np.cumsum(q_arr)))
            cursor = int(cu[-1])
            tok_seq = np.repeat(np.arange(real_b), q_arr)
            tok_pos = np.arange(cursor) - np.repeat(cu[:-1] - starts, q_arr)
            buf[v_tok[0]: v_tok[0] + cursor] = np.fromiter(
                itertools.chain.from_iterable(e.tokens for e in entries), dtype=np.int64, count=cursor)
            buf[v_pos[0]: v_pos[0] + cursor] = tok_pos
            buf[v_seq[0]: v_seq[0] + cursor] = tok_seq
            q_starts, start_positions = cu[:-1].tolist(), starts.tolist()
            for i, e in enumerate(entries):
                for w in e.want:
                    if not 0 <= w < q_lens[i]:
                        raise ValueError(f"wanted place {w} is outside the {q_lens[i]} tokens of {e.req_id!r}")
                    logit_rows.append(q_starts[i] + w)
            slot_of_seq = np.fromiter((self.cache.state_slot(e.req_id) for e in entries), dtype=np.int64, count=real_b)
            page_index = tok_pos // ps
            for g in range(len(tables)):
                rows_g = dense[g]
                if int(page_index.max()) >= rows_g.shape[1]:
                    raise ValueError("a request is longer than the cache manager's block tables")
                cols = min(width, rows_g.shape[1])
                block = buf[v_tables[g][0]: v_tables[g][0] + b * width].reshape(b, width)
                block[:real_b, :cols] = rows_g[slot_of_seq, :cols]
                block[:real_b, cols:] = -1
                pages = rows_g[slot_of_seq[tok_seq], page_index]
                if (pages < 0).any():
                    bad = entries[int(tok_seq[int(np.argmax(pages < 0))])]
                    raise ValueError(f"request {bad.req_id!r} has no page for one of positions {bad.start} to "
                                     f"{bad.start + len(bad.tokens) - 1} (never grown to there, or given back)")
                buf[v_slots[g][0]: v_slots[g][0] + cursor] = pages.astype(np.int64) * ps + tok_pos % ps
        for i, e in enumerate(entries if dense is None else ()):
            ql = q_lens[i]
            q_starts.append(cursor)
            start_positions.append(e.start)
            buf[v_tok[0] + cursor: v_tok[0] + cursor + ql] = e.tokens
            buf[v_pos[0] + cursor: v_pos[0] + cursor + ql] = np.arange(e.start, e.start + ql)
            buf[v_seq[0] + cursor: v_seq[0] + cursor + ql] = i
            for w in e.want:
                if not 0 <= w < ql:
                    raise ValueError(f"wanted place {w} is outside the {ql} tokens of {e.req_id!r}")
                logit_rows.append(cursor + w)
            for g, group_tables in enumerate(tables):
                table = group_tables[i]
                if len(table) * ps < e.start + ql:
                    raise ValueError(f"request {e.req_id!r} has no pages for positions up to "
                                     f"{e.start + ql}; call grow() first")
                pos = np.arange(e.start, e.start + ql)
                pages = np.asarray(table, dtype=np.int64)[pos // ps]
                if (pages < 0).any():
                    raise ValueError(f"request {e.req_id!r} writes to a page it gave back")
                buf[v_slots[g][0] + cursor: v_slots[g][0] + cursor + ql] = pages * ps + pos % ps
                row = v_tables[g][0] + i * width
                buf[row: row + len(table)] = table
                buf[row + len(table): row + width] = -1
            cursor += ql
        ctx_lens = [s + q for s, q in zip(start_positions, q_lens)]
        state_slots = [self.cache.state_slot(e.req_id) for e in entries]
        for j in range(pad):  # padded rows: one token at position 0 on the scratch page
            i = real_b + j
            q_starts.append(cursor)
            start_positions.append(0)
            q_lens.append(1)
            ctx_lens.append(1)
            state_slots.append(self.cache.max_requests)
            buf[v_tok[0] + cursor] = 0
            buf[v_pos[0] + cursor] = 0
            buf[v_seq[0] + cursor] = i
            logit_rows.append(cursor)
            for g, st in enumerate(self.storage.paged):
                buf[v_slots[g][0] + cursor] = st.scratch_page * ps
                row = v_tables[g][0] + i * width
                buf[row] = st.scratch_page
                buf[row + 1: row + width] = -1
            cursor += 1
        last_token_of_a_sequence = n
        if pad_to_tokens is not None:
            last_token_of_a_sequence = cursor
            if pad_tokens:
                # The tokens beyond the step's own: token 0 at position 0, their keys and values go to
                # the scratch page.  They name the next sequence as theirs (`seq_of_token`: the kernel
                # that walks tokens finds the scratch page's one key there), but that sequence, like
                # those after it, holds no tokens by `cu_q`: the kernels that walk sequences do nothing
                # for them, and their rows of the attention's output are never read.
                pos = np.arange(pad_tokens)
                buf[v_tok[0] + cursor: v_tok[0] + cursor + pad_tokens] = 0
                buf[v_pos[0] + cursor: v_pos[0] + cursor + pad_tokens] = 0
                buf[v_seq[0] + cursor: v_seq[0] + cursor + pad_tokens] = real_b
                for g, st in enumerate(self.storage.paged):
                    buf[v_slots[g][0] + cursor: v_slots[g][0] + cursor + pad_tokens] = st.scratch_page * ps + pos % ps
                cursor += pad_tokens
            for i in range(len(q_starts), b):  # sequences without tokens
                q_starts.append(last_token_of_a_sequence)
                start_positions.append(0)
                q_lens.append(0)
                ctx_lens.append(0)
                state_slots.append(self.cache.max_requests)
                for g, st in enumerate(self.storage.paged):
                    row = v_tables[g][0] + i * width
                    buf[row] = st.scratch_page
                    buf[row + 1: row + width] = -1
            logit_rows += [0] * (rows - len(logit_rows))
        buf[v_cu[0]: v_cu[0] + b] = q_starts
        buf[v_cu[0] + b] = last_token_of_a_sequence
        buf[v_ctx[0]: v_ctx[0] + b] = ctx_lens
        buf[v_state[0]: v_state[0] + b] = state_slots
        buf[v_rows[0]: v_rows[0] + rows] = logit_rows
        # the sequences by context length, the longest first: the order in which the decode attention
        # starts their blocks (with more blocks than the device runs at once the short ones fill the end)
        buf[v_order[0]: v_order[0] + b] = np.argsort(-np.asarray(ctx_lens, dtype=np.int64), kind="stable")

        self._staging_dev[:off].copy_(self._staging_host[turn][:off], non_blocking=True)
        if self._staging_events[turn] is not None:
            self._staging_events[turn].record()
            self._staging_used[turn] = True
        self.last_h2d_bytes = off * 4
        dev = self._staging_dev

        def dview(view, shape=None):
            t = dev[view[0]: view[0] + view[1]]
            return t if shape is None else t.view(*shape)

        # (of the requests that bring one token: the others are not the decode kernel's)
        ragged = self.contexts_are_ragged([c for c, ql in zip(ctx_lens[:real_b], q_lens) if ql == 1])
        if pad_to_tokens is not None:  # (a launch that serves every step that fits knows no lengths)
            ragged = tuple(0 for _ in ragged)
        groups: list[Any] = []
        for g, st in enumerate(self.storage.paged):
            groups.append(PagedGroupView(st.k, st.v, ps, st.window, dview(v_tables[g], (b, width)),
                                         width, dview(v_slots[g]), ragged[g]))
        state_dev = dview(v_state)
        for st in self.storage.state:
            groups.append(StateGroupView(st, state_dev, state_slots))
        ctx = StepContext(
            ops=self.ops, ws=self.ws, num_tokens=n, num_seqs=b,
            token_ids=dview(v_tok), positions=dview(v_pos), seq_of_token=dview(v_seq),
            cu_q=dview(v_cu), ctx_lens=dview(v_ctx), groups=groups,
            q_starts=q_starts, q_lens=q_lens, start_positions=start_positions,
            max_q_len=max(q_lens), max_ctx_len=max(ctx_lens), padded=pad_to_seqs is not None,
            ragged=ragged, decode_order=dview(v_order),
            bounds=None if pad_to_tokens is None else (n, b, width * ps),
        )
        return ctx, dview(v_rows)

    def prepare_decode(self, req_ids: list, positions: list[int], pad_to_seqs: int, table_width: int):
        """Pack a decode step whose token ids are not known yet (they are being sampled on the
        device right now) into a pinned buffer, without copying it.  Returns a handle for
        :meth:`commit_prepared`, which fills in the tokens and starts the copy.  Every entry
        wants its logits."""
        entries = [StepEntry(r, [0], p, [0]) for r, p in zip(req_ids, positions)]
        return self._build_decode_context(entries, pad_to_seqs, table_width, views=False, defer=True)

    def commit_prepared(self, handle, tokens) -> None:
        """``tokens``: the step's token ids as a list, or as a 32-bit device tensor (the ids a
        sampling kernel is still writing: they go from device to device, in stream order)."""
        turn, off, tok_at, count = handle
        on_device = not isinstance(tokens, (list, tuple))
        if not on_device:
            self._staging_host[turn][tok_at: tok_at + count] = self._torch.tensor(tokens, dtype=self._torch.int32)
        self._staging_dev[:off].copy_(self._staging_host[turn][:off], non_blocking=True)
        if on_device:
            self._staging_dev[tok_at: tok_at + count].copy_(tokens[:count], non_blocking=True)
        if self._staging_events[turn] is not None:
            self._staging_events[turn].record()
            self._staging_used[turn] = True
        self.last_h2d_bytes = off * 4

    def _build_decode_context(self, entries: list[StepEntry], pad_to_seqs: int | None,
                              table_width: int | None, views: bool = True, defer: bool = False):
        """The same packing for a step of single tokens, without a Python loop over what the
        entries hold: block-table rows are gathered from the cache manager's dense copy."""
        import numpy as np

        ps, cache = self.page_size, self.cache
        real_b = len(entries)
        b = max(pad_to_seqs or 0, real_b)
        pad = b - real_b
        positions = np.fromiter((e.start for e in entries), dtype=np.int64, count=real_b)
        state_slots = [cache.state_slot(e.req_id) for e in entries]
        slots_arr = np.asarray(state_slots, dtype=np.int64)
        logit_rows = [i for i, e in enumerate(entries) if e.want]
        if any(len(e.want) > 1 or (e.want and e.want[0] != 0) for e in entries):
            raise ValueError("a single-token entry can only want place 0")
        logit_rows += list(range(real_b, b))
        rows = len(logit_rows)
        page_index = positions // ps
        width = max(table_width or 1, int(page_index.max()) + 1)
        self._ensure_staging(self._staging_ints(b, b, rows, width))
        turn, buf = self._next_host_buffer()
        off = 0

        def take(count: int):
            nonlocal off
            view = (off, count)
            off += _align4(count)
            return view

        v_tok, v_pos, v_seq = take(b), take(b), take(b)
        v_cu, v_ctx, v_state, v_rows = take(b + 1), take(b), take(b), take(rows)
        v_order = take(b)
        v_slots = [take(b) for _ in cache.paged_groups]
        v_tables = [take(b * width) for _ in cache.paged_groups]
        buf[v_tok[0]: v_tok[0] + real_b] = [e.tokens[0] for e in entries]
        buf[v_pos[0]: v_pos[0] + real_b] = positions
        buf[v_seq[0]: v_seq[0] + b] = np.arange(b)
        buf[v_cu[0]: v_cu[0] + b + 1] = np.arange(b + 1)
        buf[v_ctx[0]: v_ctx[0] + real_b] = positions + 1
        buf[v_state[0]: v_state[0] + real_b] = slots_arr
        buf[v_rows[0]: v_rows[0] + rows] = logit_rows
        # (the sequences by context length, the longest first; the padding's last: see build_context)
        buf[v_order[0]: v_order[0] + real_b] = np.argsort(-positions, kind="stable")
        if pad:
            buf[v_order[0] + real_b: v_order[0] + b] = np.arange(real_b, b)
            buf[v_tok[0] + real_b: v_tok[0] + b] = 0
            buf[v_pos[0] + real_b: v_pos[0] + b] = 0
            buf[v_ctx[0] + real_b: v_ctx[0] + b] = 1
            buf[v_state[0] + real_b: v_state[0] + b] = cache.max_requests
        for g, st in enumerate(self.storage.paged):
            dense = cache.table_rows[g]
            cols = min(width, dense.shape[1])
            block = buf[v_tables[g][0]: v_tables[g][0] + b * width].reshape(b, width)
            block[:real_b, :cols] = dense[slots_arr, :cols]
            if cols < width:
                block[:real_b, cols:] = -1
            if int(page_index.max()) >= dense.shape[1]:
                raise ValueError("a request is longer than the cache manager's block tables")
            pages = dense[slots_arr, page_index]
            if (pages < 0).any():
                bad = entries[int(np.argmax(pages < 0))]
                raise ValueError(f"request {bad.req_id!r} has no page for position {bad.start}; "
                                 "call grow() first")
            buf[v_slots[g][0]: v_slots[g][0] + real_b] = pages * ps + positions % ps
            if pad:
                block[real_b:, 0] = st.scratch_page
                block[real_b:, 1:] = -1
                buf[v_slots[g][0] + real_b: v_slots[g][0] + b] = st.scratch_page * ps
        if defer:  # the tokens come later: see commit_prepared
            return (turn, off, v_tok[0], real_b)
        self._staging_dev[:off].copy_(self._staging_host[turn][:off], non_blocking=True)
        if self._staging_events[turn] is not None:
            self._staging_events[turn].record()
            self._staging_used[turn] = True
        self.last_h2d_bytes = off * 4
        if not views:  # a captured launch sequence already holds these addresses
            return None, None
        dev = self._staging_dev

        def dview(view, shape=None):
            t = dev[view[0]: view[0] + view[1]]
            return t if shape is None else t.view(*shape)

        ragged = self.contexts_are_ragged((positions + 1).tolist())
        groups: list[Any] = []
        for g, st in enumerate(self.storage.paged):
            groups.append(PagedGroupView(st.k, st.v, ps, st.window, dview(v_tables[g], (b, width)),
                                         width, dview(v_slots[g]), ragged[g]))
        state_dev = dview(v_state)
        all_slots = state_slots + [cache.max_requests] * pad
        for st in self.storage.state:
            groups.append(StateGroupView(st, state_dev, all_slots))
        start_positions = positions.tolist() + [0] * pad
        ctx = StepContext(
            ops=self.ops, ws=self.ws, num_tokens=b, num_seqs=b,
            token_ids=dview(v_tok), positions=dview(v_pos), seq_of_token=dview(v_seq),
            cu_q=dview(v_cu), ctx_lens=dview(v_ctx), groups=groups,
            q_starts=list(range(b)), q_lens=[1] * b, start_positions=start_positions,
            max_q_len=1, max_ctx_len=int(positions.max()) + 1, padded=pad_to_seqs is not None,
            ragged=ragged, decode_order=dview(v_order),
        )
        return ctx, dview(v_rows)

    def reset_fresh_state(self, ctx: StepContext) -> None:
        """A request whose tokens start at position 0 starts from a zero state."""
        if not self.storage.state:
            return
        torch = self._torch
        slots = [s for s, p in zip(ctx.groups[len(self.storage.paged)].slots_host,
                                   ctx.start_positions) if p == 0]
        if not slots:
            return
        index = torch.tensor(slots, dtype=torch.long, device=self.device)
        for st in self.storage.state:
            st.index_fill_(1, index, 0.0)

    def step(self, entries: list[StepEntry]):
        """Run the entries as one batch; return ``[wanted, vocab]`` 32-bit logits in the order
        of the entries and of their ``want`` lists, or None when nothing is wanted."""
        ctx, logit_rows = self.build_context(entries)
        self.reset_fresh_state(ctx)
        return self.model.forward(ctx, logit_rows)


def make_runner(model: Model, ops, device, page_size: int, num_pages: int, max_requests: int,
                max_tokens_per_step: int) -> ModelRunner:
    """Cache manager, device storage and step function for ``model``."""
    cache = CacheManager(model.paged_groups, model.state_groups, num_pages, page_size, max_requests)
    storage = CacheStorage(cache, model.env.torch_dtype, device)
    return ModelRunner(model, cache, storage, ops, device, max_tokens_per_step, max_requests)
