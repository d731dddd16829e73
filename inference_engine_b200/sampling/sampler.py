"""From a step's logits to one token per finished row, on the device.

One kernel launch serves all rows: greedy rows take the argmax (lowest index on ties, as
``torch.argmax``), the others are drawn at their temperature after the repetition penalty and
the top-k / top-p / min-p cut-offs, in the reference's order (engine/runtime/sampler.py:10-45).
Randomness is counter-based: row ``r`` uses (its request's seed, how many tokens the request
has produced), so a request's tokens do not depend on its neighbours in the batch.  The
reference draws with ``torch.multinomial`` from one generator per request
(engine/runtime/engine.py:156-157); the two agree in distribution, not bit for bit.
"""

from __future__ import annotations

from typing import Any, Sequence as Seq


class Sampler:
    def __init__(self, ops, device, vocab_size: int) -> None:
        import torch

        self.ops, self.device, self.vocab_size, self.torch = ops, device, vocab_size, torch
        # Two sets of output buffers in turn: the engine may start the next step, which reads
        # this step's tokens on the device, and its sampling before it has fetched these.
        self._tokens = [torch.empty(0, dtype=torch.int32, device=device) for _ in range(2)]
        self._host = [None, None]     # pinned copies of the tokens
        self._err_host = [None, None]  # pinned copies of the kernels' error word, fetched with the tokens
        self._events = [None, None]
        self._turn = 0
        self._param_dev, self._param_cap, self._param_key, self._param_draws, self._param_turn = None, 0, None, [], 0
        self._bits_host, self._bits_dev, self._bits_turn = None, None, 0
        self._masks: dict = {}  # request key -> (ids of its history already in the mask, the mask)

    def _out(self, rows: int):
        i = self._turn = 1 - self._turn
        if self._tokens[i].numel() < rows:
            torch = self.torch
            n = max(rows, 64)
            self._tokens[i] = torch.empty(n, dtype=torch.int32, device=self.device)
            pinned = torch.device(self.device).type == "cuda"
            self._host[i] = torch.empty(n, dtype=torch.int32, pin_memory=pinned)
            self._err_host[i] = torch.zeros(4, dtype=torch.int32, pin_memory=pinned)
            self._events[i] = torch.cuda.Event() if pinned else None
        return i, self._tokens[i][:rows]

    def sample(self, logits, params: Seq[Any], seeds: Seq[int], draws: Seq[int],
               histories: Seq[Seq[int]] | None = None, history_keys: Seq[Any] | None = None):
        """``logits``: 32-bit ``[R, vocab]``.  ``params[r]``: the row's SamplingParams,
        ``seeds[r]``/``draws[r]``: its request's seed and the number of tokens it has already
        produced; ``histories[r]``: the ids the repetition penalty looks at.
        Returns ``(tokens, logprobs)``: a list of ints and a list of floats or None."""
        return self.collect(self.launch(logits, params, seeds, draws, histories, history_keys))

    def launch(self, logits, params, seeds, draws, histories=None, history_keys=None):
        """Start the sampling kernel; :meth:`collect` waits for it and fetches the tokens.
        ``history_keys[r]`` (optional): something that names row r's request from step to step,
        so that its history's bit mask is extended by the new ids instead of built again."""
        torch = self.torch
        rows = logits.shape[0]
        turn, out = self._out(rows)
        want_logprobs = any(p.logprobs for p in params)
        logprob = torch.empty(rows, dtype=torch.float32, device=self.device) if want_logprobs else None
        if all(p.greedy and p.repetition_penalty == 1.0 for p in params):
            self.ops.sample(logits, out, logprob=logprob)
        else:
            kwargs = self._row_parameters(params, seeds, draws)
            if any(p.repetition_penalty != 1.0 for p in params):
                kwargs["seen_bits"] = self._seen_bits(params, histories, history_keys)
            self.ops.sample(logits, out, logprob=logprob, **kwargs)
        # the tokens start on their way to the host right behind the kernel
        host = self._host[turn][:rows]
        host.copy_(out, non_blocking=True)
        # ... and with them the word in which the step's kernels report an index out of range or
        # a wait that ran out (16 bytes; no extra wait: it is read when the tokens are)
        err_word = getattr(self.ops, "err", None)
        err_host = None
        if err_word is not None:
            err_host = self._err_host[turn]
            err_host.copy_(err_word, non_blocking=True)
        if self._events[turn] is not None:
            self._events[turn].record()
        return out, logprob, host, self._events[turn], err_host

    # The rows' parameters live in one device buffer.  They reach it as one copy from pinned
    # memory (a copy from pageable memory would make the host wait for the stream, and with it
    # for the step that is still running); while the same requests decode on, nothing but the
    # draw counters changes, and those are advanced on the device.
    RING = 4

    def _row_parameters(self, params, seeds, draws) -> dict:
        import numpy as np

        torch = self.torch
        rows = len(params)
        settings = tuple((p.temperature, p.top_k, p.top_p, p.min_p, p.repetition_penalty) for p in params)
        key = (settings, tuple(seeds))
        cap = self._param_cap
        if rows > cap or self._param_dev is None:
            cap = self._param_cap = max(64, 2 * rows)
            pinned = torch.device(self.device).type == "cuda"
            self._param_dev = torch.zeros(9 * cap, dtype=torch.int32, device=self.device)
            self._param_host = [torch.zeros(9 * cap, dtype=torch.int32, pin_memory=pinned) for _ in range(self.RING)]
            self._param_events = [torch.cuda.Event() if pinned else None for _ in range(self.RING)]
            self._param_used = [False] * self.RING
            self._param_key = None
        dev = self._param_dev
        section = lambda i, width=1: dev[i * cap: (i + width) * cap]  # noqa: E731
        views = {
            "temperature": section(0).view(torch.float32)[:rows], "top_k": section(1)[:rows],
            "top_p": section(2).view(torch.float32)[:rows], "min_p": section(3).view(torch.float32)[:rows],
            "penalty": section(4).view(torch.float32)[:rows],
            "seeds": section(5, 2).view(torch.int64)[:rows], "draws": section(7, 2).view(torch.int64)[:rows],
        }
        if key == self._param_key and list(draws) == [d + 1 for d in self._param_draws]:
            views["draws"].add_(1)  # the same requests, one token further
        else:
            turn = self._param_turn = (self._param_turn + 1) % self.RING
            if self._param_used[turn] and self._param_events[turn] is not None:
                self._param_events[turn].synchronize()  # the copy that last read this buffer has run
            host = self._param_host[turn].numpy()
            host[0 * cap: 0 * cap + rows] = np.asarray([s[0] for s in settings], dtype=np.float32).view(np.int32)
            host[1 * cap: 1 * cap + rows] = np.asarray([s[1] for s in settings], dtype=np.int32)
            host[2 * cap: 2 * cap + rows] = np.asarray([s[2] for s in settings], dtype=np.float32).view(np.int32)
            host[3 * cap: 3 * cap + rows] = np.asarray([s[3] for s in settings], dtype=np.float32).view(np.int32)
            host[4 * cap: 4 * cap + rows] = np.asarray([s[4] for s in settings], dtype=np.float32).view(np.int32)
            host[5 * cap: 5 * cap + 2 * rows] = np.asarray([s & 0x7FFFFFFFFFFFFFFF for s in seeds], dtype=np.int64).view(np.int32)
            host[7 * cap: 7 * cap + 2 * rows] = np.asarray(list(draws), dtype=np.int64).view(np.int32)
            dev.copy_(self._param_host[turn], non_blocking=True)
            if self._param_events[turn] is not None:
                self._param_events[turn].record()
                self._param_used[turn] = True
            self._param_key = key
        self._param_draws = list(draws)
        kwargs = {"temperature": views["temperature"], "seeds": views["seeds"], "draws": views["draws"]}
        if any(s[1] > 0 for s in settings):
            kwargs["top_k"] = views["top_k"]
        if any(s[2] < 1.0 for s in settings):
            kwargs["top_p"] = views["top_p"]
        if any(s[3] > 0.0 for s in settings):
            kwargs["min_p"] = views["min_p"]
        if any(s[4] != 1.0 for s in settings):
            kwargs["penalty"] = views["penalty"]
        return kwargs

    def collect(self, pending):
        out, logprob, host, event, err_host = pending
        if event is not None:
            event.synchronize()  # the step's one wait for the device: until its tokens have arrived
        if err_host is not None and int(err_host[0]):
            self.ops.raise_reported(err_host.tolist())  # these tokens cannot be trusted
        tokens = host.tolist()
        return tokens, (logprob.tolist() if logprob is not None else None)

    def _seen_bits(self, params, histories, keys=None):
        """One bit per vocabulary entry and row: set where the id occurs in the row's history.
        A history only grows (and its request's key stays), so a row's mask from the last step
        is extended by the ids that are new; the masks go to the device as one copy from pinned
        memory."""
        import numpy as np

        torch = self.torch
        rows, words = len(params), (self.vocab_size + 31) // 32
        if self._bits_host is None or self._bits_host[0].shape[0] < rows:
            cap = max(8, 2 * rows)
            pinned = torch.device(self.device).type == "cuda"
            self._bits_host = [torch.zeros(cap, words, dtype=torch.int32, pin_memory=pinned) for _ in range(self.RING)]
            self._bits_events = [torch.cuda.Event() if pinned else None for _ in range(self.RING)]
            self._bits_used = [False] * self.RING
            self._bits_dev = torch.zeros(cap, words, dtype=torch.int32, device=self.device)
        turn = self._bits_turn = (self._bits_turn + 1) % self.RING
        if self._bits_used[turn] and self._bits_events[turn] is not None:
            self._bits_events[turn].synchronize()
        host = self._bits_host[turn].numpy().view(np.uint32)
        if len(self._masks) > 4096:  # requests long gone
            self._masks.clear()
        for r, (p, hist) in enumerate(zip(params, histories or [])):
            if p.repetition_penalty == 1.0 or not hist:
                host[r] = 0
                continue
            key = keys[r] if keys is not None else None
            known, mask = self._masks.get(key, (0, None)) if key is not None else (0, None)
            if mask is None or known > len(hist):
                known, mask = 0, np.zeros(words, dtype=np.uint32)
            ids = np.asarray(hist[known:], dtype=np.int64)
            if ids.size:
                np.bitwise_or.at(mask, ids >> 5, (np.uint32(1) << (ids & 31).astype(np.uint32)))
            if key is not None:
                self._masks[key] = (len(hist), mask)
            host[r] = mask
        dev = self._bits_dev[:rows]
        dev.copy_(self._bits_host[turn][:rows], non_blocking=True)
        if self._bits_events[turn] is not None:
            self._bits_events[turn].record()
            self._bits_used[turn] = True
        return dev

    def top_logprobs(self, logits_row, k: int) -> list[tuple[int, float]]:
        """The ``k`` most likely alternatives of one row with their log-probabilities
        (engine/runtime/engine.py:283-298)."""
        lp = logits_row.float().log_softmax(-1)
        top = lp.topk(k)
        return list(zip(top.indices.tolist(), top.values.tolist()))
