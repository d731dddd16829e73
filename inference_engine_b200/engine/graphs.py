"""Decode steps, and short steps that hold prompt portions, as captured launch sequences (CUDA graphs).

A decode-only step launches a hundred and more small kernels; at small batches their launch
cost is a large part of the step.  For a few batch sizes (buckets) the whole forward pass is
captured once and replayed: the step's index data is copied into the same staging addresses,
padded up to the bucket with rows that read and write the cache's scratch page, and every
kernel takes lengths and tables from device memory, so one capture serves every context
length.  Bucket sizes are the reference's (engine/runtime/cuda_graphs.py:20-108).

The block tables' row stride is fixed in a capture.  A stride for the longest context the
engine allows (8,192 entries of 16 tokens at Llama 3.2's 131,072 positions) would make every
step copy megabytes of table to the device for contexts of a few hundred tokens, so the
stride is part of what a capture is keyed by: the smallest of 64, 128, 256, ... entries
(up to the engine's limit) that holds the step's longest context.

Steps with prompt portions (`MixedGraphs`): an eager step costs the host about 13 us per kernel,
1.9 ms for the sixteen layers of the 1B shape, whatever the step holds; up to a few hundred
tokens the device needs half of that (a 384-token step 2.06 ms eager, 1.31 captured; 512 tokens 2.25
and 1.62; 1,024 tokens 2.59 and 2.42: beyond that the device is the bound and steps stay eager).  Such steps are captured too, per (tokens, sequences,
wanted rows, block-table stride), each rounded up to a bucket: the tokens beyond the step's own
belong to no sequence (their keys and values go to the cache's scratch page), the sequences
beyond the step's own hold no tokens, and the attention is launched for the most query tiles any step within the bounds can
have (`StepContext.bounds`).  The reference captures such steps piecewise, around an eager
attention (engine/runtime/cuda_graphs.py:113-228); here the attention kernels take every length
from device memory, so the whole step is one launch sequence.
"""

from __future__ import annotations

BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)
TOKEN_BUCKETS = (8, 16, 32, 64, 128, 256, 384, 512, 768, 1024)  # captured steps with prompt portions: up to this many tokens
SEQ_BUCKETS = (4, 16, 64)  # ... and their sequences, up to the largest decode bucket


def _capture(torch, graph, forward):
    """Record ``forward()``'s launches into ``graph``.  The garbage collector stays off meanwhile:
    an object it frees may own captured launch sequences or device memory, and giving those back
    while a stream is capturing makes the capture invalid.  (It is not run beforehand either: a
    full collection costs tens of milliseconds on a process of this size, as much as the capture.)"""
    import gc

    was_enabled = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.graph(graph):
            return forward()
    finally:
        if was_enabled:
            gc.enable()


class DecodeGraphs:
    def __init__(self, runner, max_num_seqs: int, table_width: int) -> None:
        import torch

        self.torch, self.runner = torch, runner
        self.table_width = table_width
        self.buckets = [b for b in BUCKETS if b <= max_num_seqs]
        if not self.buckets or self.buckets[-1] < max_num_seqs:
            self.buckets.append(max_num_seqs)
        # one capture per (bucket, whether the contexts' lengths differ much: the attention is
        # launched differently for the two, block-table row stride)
        self._graphs: dict[tuple, tuple] = {}
        self._version = None
        self.replays = 0

    def bucket_for(self, num_seqs: int) -> int | None:
        for b in self.buckets:
            if b >= num_seqs:
                return b
        return None

    MIN_WIDTH = 64

    def width_for(self, last_position: int) -> int:
        """The block-table row stride for a step whose longest request reaches ``last_position``."""
        pages = last_position // self.runner.page_size + 1
        width = self.MIN_WIDTH
        while width < pages:
            width *= 2
        return max(min(width, self.table_width), pages)

    def kernels_per_replay(self, num_seqs: int) -> int:
        """How many of the engine's own kernels one replay for ``num_seqs`` sequences launches."""
        bucket = self.bucket_for(num_seqs)
        for (size, *_), entry in self._graphs.items():
            if size == bucket:
                return entry[2]
        return 0

    def prepare(self, req_ids: list, positions: list[int]):
        """Pack the next decode step ahead of time (while the device still works on this one)
        if a captured launch sequence for its batch size exists; None otherwise."""
        bucket = self.bucket_for(len(req_ids))
        width = self.width_for(max(positions))
        key = (bucket, self.runner.contexts_are_ragged([p + 1 for p in positions]), width)
        if bucket is None or key not in self._graphs or self._version != self.runner.ws.version:
            return None
        if width > self.table_width:
            return None
        handle = self.runner.prepare_decode(req_ids, positions, bucket, width)
        if self._version != self.runner.ws.version:
            return None
        return (key, handle)

    def run_prepared(self, prepared, tokens, count: int | None = None):
        """Fill the sampled tokens (a list, or a device tensor of which the first ``count`` are
        taken) into a step packed by :meth:`prepare` and replay it."""
        key, handle = prepared
        if key not in self._graphs or self._version != self.runner.ws.version:
            return None
        self.runner.commit_prepared(handle, tokens)
        graph, logits, _ = self._graphs[key]
        graph.replay()
        self.replays += 1
        return logits[: len(tokens) if count is None else count]

    def can_run(self, entries) -> bool:
        if not entries or any(len(e.tokens) != 1 for e in entries):
            return False
        if self.bucket_for(len(entries)) is None:
            return False
        return self.width_for(max(e.start for e in entries)) <= self.table_width

    def run(self, entries):
        """Returns the ``[len(entries), vocab]`` logits of a decode-only step (every entry
        must want its one token)."""
        torch, runner = self.torch, self.runner
        bucket = self.bucket_for(len(entries))
        if self._version != runner.ws.version:  # a buffer moved: captured addresses are stale
            self._graphs.clear()
            self._version = runner.ws.version
        width = self.width_for(max(e.start for e in entries))
        key = (bucket, self.runner.contexts_are_ragged([e.start + 1 for e in entries]), width)
        captured = key in self._graphs
        ctx, rows = runner.build_context(entries, pad_to_seqs=bucket, table_width=width,
                                         views=not captured)
        if self._version != runner.ws.version:  # the staging buffer itself had to grow
            self._graphs.clear()
            self._version = runner.ws.version
            captured = False
            ctx, rows = runner.build_context(entries, pad_to_seqs=bucket, table_width=width)
        if not captured:
            # Run once outside a capture (buffers get allocated, libraries initialised) ...
            stream = torch.cuda.Stream()
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                runner.model.forward(ctx, rows)
            torch.cuda.current_stream().wait_stream(stream)
            torch.cuda.synchronize()
            if self._version != runner.ws.version:
                self._graphs.clear()
                self._version = runner.ws.version
                ctx, rows = runner.build_context(entries, pad_to_seqs=bucket, table_width=width)
            # ... then record the same launches.
            graph = torch.cuda.CUDAGraph()
            before = getattr(runner.ops, "launches", 0)
            logits = _capture(torch, graph, lambda: runner.model.forward(ctx, rows))
            self._graphs[key] = (graph, logits, getattr(runner.ops, "launches", 0) - before)
        graph, logits, _ = self._graphs[key]
        graph.replay()
        self.replays += 1
        return logits[: len(entries)]


class MixedGraphs:
    """Short steps that hold prompt portions (beside decode tokens or not) as captured launch
    sequences; see the module's text.  Shares the decode captures' bucket list and stride rule."""

    def __init__(self, decode_graphs: DecodeGraphs, max_tokens: int = TOKEN_BUCKETS[-1]) -> None:
        self.torch, self.runner, self.decode = decode_graphs.torch, decode_graphs.runner, decode_graphs
        self.token_buckets = [t for t in TOKEN_BUCKETS if t <= max_tokens]
        if max_tokens < TOKEN_BUCKETS[-1] and max_tokens not in self.token_buckets:
            self.token_buckets.append(max_tokens)  # (the engine's own limit of tokens per step)
        largest = decode_graphs.buckets[-1] + 1  # (all the engine's sequences and the one for the padding)
        self.seq_buckets = [b for b in SEQ_BUCKETS if b < largest] + [largest]
        self._graphs: dict[tuple, tuple] = {}
        self._version = None
        self.replays = 0

    def _key(self, entries):
        """(tokens, sequences, wanted rows, block-table stride) of the launch that serves these
        entries, or None if none does."""
        tokens = sum(len(e.tokens) for e in entries)
        t_b = next((t for t in self.token_buckets if t >= tokens), None)
        if t_b is None:
            return None
        # (one sequence more than the step's own: the one that takes the tokens beyond them; a
        # sequence without tokens and a wanted row too many cost next to nothing, a capture costs
        # memory and a first step of tens of milliseconds: few, coarse sizes)
        s_b = next((b for b in self.seq_buckets if b >= len(entries) + 1), None)
        if s_b is None:
            return None
        wanted = sum(len(e.want) for e in entries)
        r_b = s_b if wanted <= s_b else self.decode.bucket_for(wanted)
        if r_b is None:
            return None
        ps = self.runner.page_size
        pages = max((e.start + len(e.tokens) - 1) // ps + 1 for e in entries)
        width = self.decode.MIN_WIDTH
        while width < pages:
            width *= 2
        if width > self.decode.table_width:
            width = self.decode.table_width
            if width < pages:
                return None
        return t_b, s_b, r_b, width

    def can_run(self, entries) -> bool:
        return bool(entries) and any(len(e.tokens) > 1 for e in entries) and self._key(entries) is not None

    def run(self, entries):
        """Returns the ``[wanted, vocab]`` logits of the step, in the order of the entries and
        of their ``want`` lists, or None when nothing is wanted."""
        torch, runner = self.torch, self.runner
        if self._version != runner.ws.version:  # a buffer moved: captured addresses are stale
            self._graphs.clear()
            self._version = runner.ws.version
        key = self._key(entries)
        t_b, s_b, r_b, width = key
        wanted = sum(len(e.want) for e in entries)

        def build():
            return runner.build_context(entries, pad_to_seqs=s_b, table_width=width, pad_to_tokens=t_b,
                                        pad_to_rows=r_b)

        ctx, rows = build()
        if self._version != runner.ws.version:  # the staging buffer itself had to grow
            self._graphs.clear()
            self._version = runner.ws.version
            ctx, rows = build()
        if ctx.bounds != (t_b, s_b, width * runner.page_size):
            raise RuntimeError(f"a step packed for {ctx.bounds} cannot replay the launch captured for {key}")
        if key not in self._graphs:
            # Run once outside a capture (buffers get allocated, libraries initialised) ...
            stream = torch.cuda.Stream()
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                runner.model.forward(ctx, rows)
            torch.cuda.current_stream().wait_stream(stream)
            torch.cuda.synchronize()
            if self._version != runner.ws.version:
                self._graphs.clear()
                self._version = runner.ws.version
                ctx, rows = build()
            # ... then record the same launches.
            graph = torch.cuda.CUDAGraph()
            logits = _capture(torch, graph, lambda: runner.model.forward(ctx, rows))
            self._graphs[key] = (graph, logits)
        graph, logits = self._graphs[key]
        graph.replay()
        self.replays += 1
        return logits[:wanted] if wanted else None
