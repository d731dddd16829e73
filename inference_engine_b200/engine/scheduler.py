"""Continuous batching with a token budget, chunked prefill and recompute preemption.

The decisions are the reference's (engine/runtime/scheduler.py:74-216):

* every step has ``max_num_batched_tokens`` tokens to give out;
* running requests go first, oldest first: a decoding request takes one token, a request
  part-way through its prompt takes the next portion (all that is left if it fits the
  budget, else the budget; without chunked prefill a prompt runs whole or waits);
* what is left admits waiting requests, first come first served, never skipping the head;
* when the pages run out while a running request has to grow, the newest running request
  that has not been scheduled yet in this step is preempted (the request itself if there is
  none): it gives back all its pages and its state slot, forgets what it computed, and goes
  to the front of the waiting queue; later it is prefilled again over its prompt and the
  tokens it had produced, and samples only at the end;
* a waiting request holds no page and no slot.

Bookkeeping: ``seq.num_computed`` tokens of ``seq.all_ids`` are in the cache; a step feeds
``all_ids[num_computed : num_computed + n]``; a token is sampled only when that reaches the
end of the sequence.  No torch here.
"""

from __future__ import annotations

import enum
from collections import deque
from dataclasses import dataclass, field
from typing import Any

from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams


class SeqStatus(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


@dataclass(eq=False)
class Sequence:
    seq_id: int
    request_id: str
    prompt_ids: list[int]
    params: SamplingParams
    output_ids: list[int] = field(default_factory=list)
    num_computed: int = 0
    status: SeqStatus = SeqStatus.WAITING
    finish_reason: str | None = None
    num_preemptions: int = 0
    seed: int = 0  # the request's sampling seed (its own, or drawn when it was added)
    processor: Any = None

    @property
    def all_ids(self) -> list[int]:
        return self.prompt_ids + self.output_ids

    @property
    def length(self) -> int:
        return len(self.prompt_ids) + len(self.output_ids)

    @property
    def num_new_tokens(self) -> int:
        return self.length - self.num_computed


@dataclass
class ScheduledBatch:
    seqs: list[Sequence]
    num_tokens: list[int]  # tokens fed for each sequence in this step

    @property
    def total_tokens(self) -> int:
        return sum(self.num_tokens)


class Scheduler:
    def __init__(self, cache: CacheManager, max_num_seqs: int = 64,
                 max_num_batched_tokens: int = 4096, enable_chunked_prefill: bool = True) -> None:
        if max_num_batched_tokens < max_num_seqs:
            raise ValueError("max_num_batched_tokens must be >= max_num_seqs (one per decode)")
        if max_num_seqs > cache.max_requests:
            raise ValueError("max_num_seqs exceeds the cache manager's state slots")
        self.cache = cache
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.enable_chunked_prefill = enable_chunked_prefill
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []
        self.num_preemptions = 0

    @property
    def capacity_tokens(self) -> int:
        return self.cache.capacity_tokens

    def add(self, seq: Sequence) -> None:
        """Queue a request.  One that could never fit the cache by itself is refused."""
        longest = len(seq.prompt_ids) + seq.params.max_tokens
        if longest > self.capacity_tokens:
            raise ValueError(f"prompt + max_tokens = {longest} tokens exceeds the KV cache "
                             f"({self.capacity_tokens} tokens)")
        self.waiting.append(seq)

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    def abort(self, request_id: str) -> Sequence | None:
        for queue in (self.waiting, self.running):
            for seq in list(queue):
                if seq.request_id == request_id:
                    queue.remove(seq)
                    self.finish(seq, "abort")
                    return seq
        return None

    def finish(self, seq: Sequence, reason: str | None) -> None:
        seq.status, seq.finish_reason = SeqStatus.FINISHED, reason
        if seq in self.running:
            self.running.remove(seq)
        self.cache.free(seq.seq_id)  # pages and state slot, in the same step

    # --- one step ---------------------------------------------------------------------------

    def schedule(self) -> ScheduledBatch | None:
        budget = self.max_num_batched_tokens
        seqs: list[Sequence] = []
        counts: list[int] = []

        # 1. Running requests, oldest first; preempt the newest when pages run out.
        queue = list(self.running)
        kept: list[Sequence] = []
        while queue and budget > 0:
            seq = queue.pop(0)
            n = self._portion(seq, budget)
            if n == 0:
                kept.append(seq)
                continue
            target = seq.num_computed + n
            while not self.cache.try_grow(seq.seq_id, seq.num_computed, target):
                victim = queue.pop() if queue else seq
                self._preempt(victim)
                if victim is seq:
                    break
            else:
                kept.append(seq)
                seqs.append(seq)
                counts.append(n)
                budget -= n
        kept.extend(queue)  # no budget left for these in this step
        self.running = kept

        # 2. Admit waiting requests with what is left, in order of arrival.
        while self.waiting and budget > 0 and len(self.running) < self.max_num_seqs:
            seq = self.waiting[0]
            n = self._portion(seq, budget)
            if n == 0 or not self.cache.can_admit():
                break
            self.cache.add_request(seq.seq_id)
            if not self.cache.can_grow(seq.seq_id, seq.num_computed, seq.num_computed + n):
                self.cache.free(seq.seq_id)  # a waiting request holds nothing
                break
            self.cache.grow(seq.seq_id, seq.num_computed, seq.num_computed + n)
            self.waiting.popleft()
            seq.status = SeqStatus.RUNNING
            self.running.append(seq)
            seqs.append(seq)
            counts.append(n)
            budget -= n
        return ScheduledBatch(seqs, counts) if seqs else None

    def _portion(self, seq: Sequence, budget: int) -> int:
        """Tokens to feed ``seq`` in this step within ``budget`` (0 = wait)."""
        n = seq.num_new_tokens
        if n <= budget:
            return n
        if self.enable_chunked_prefill:
            return budget
        # Without chunking a prompt runs whole; one larger than the whole budget runs alone.
        return n if budget == self.max_num_batched_tokens else 0

    def _preempt(self, seq: Sequence) -> None:
        self.cache.free(seq.seq_id)
        seq.num_computed = 0
        seq.status = SeqStatus.WAITING
        seq.num_preemptions += 1
        self.num_preemptions += 1
        if seq in self.running:
            self.running.remove(seq)
        self.waiting.appendleft(seq)  # newest victims first, so the oldest ends up in front
