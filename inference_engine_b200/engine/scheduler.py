"""Continuous batching: who runs in the next step, and with how many tokens.

The scheduler is a planner and a committer.  ``plan()`` looks at the queues and at the cache
manager's free pages and decides, changing nothing: which running requests get tokens, which
are preempted to make room, which waiting requests are admitted.  ``commit(plan)`` carries it
out (pages taken and given back, queues updated).  ``schedule()`` is both.  Because planning
is free of side effects the engine can also ask ahead of time, while the device is busy,
whether the next step will be the same requests one position further
(``plan_steady_decode``), and pack that step early.

The decisions are those of the reference's scheduler (engine/runtime/scheduler.py:74-216):

* a step gives out at most ``max_num_batched_tokens`` tokens;
* running requests are served first, oldest first: all their pending ids if the budget
  allows (one id while decoding), else the rest of the budget; with chunked prefill off a
  prompt is never cut: it runs whole, or waits until it has a whole step's budget to itself;
* if the cache cannot hold a running request's next ids, the newest running request that has
  not been served in this step loses its place (the request itself if no newer one is left):
  pages and state slot go back, it forgets what it computed, keeps what it produced, and
  queues up in front of the waiting requests, older victims before newer ones;
* what is left of the budget admits waiting requests in order of arrival; the first one that
  does not fit (tokens, pages, state slots, ``max_num_seqs``) ends admission: nobody overtakes;
* a waiting request holds neither pages nor a slot.

No torch here.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from ..cache.manager import CacheManager
from .request import SeqStatus, Sequence

__all__ = ["Scheduler", "SeqStatus", "Sequence", "StepPlan"]


@dataclass
class StepPlan:
    """One step as decided: ``seqs[i]`` is fed ``num_tokens[i]`` ids (running requests first,
    then the newly admitted).  ``preempted`` lists who loses their place, in the order in
    which they lose it (newest first); ``admitted`` who comes in from the waiting queue."""

    seqs: list[Sequence] = field(default_factory=list)
    num_tokens: list[int] = field(default_factory=list)
    preempted: list[Sequence] = field(default_factory=list)
    admitted: list[Sequence] = field(default_factory=list)

    @property
    def total_tokens(self) -> int:
        return sum(self.num_tokens)

    def grant(self, seq: Sequence, count: int) -> None:
        self.seqs.append(seq)
        self.num_tokens.append(count)

    def is_decode_of(self, seqs: list[Sequence]) -> bool:
        """Exactly these requests, one token each, nobody moved."""
        return (not self.preempted and not self.admitted and self.seqs == seqs
                and all(n == 1 for n in self.num_tokens))


class _PageLedger:
    """Free pages per cache group and free state slots as they would stand while a plan is
    drawn up: reservations and give-backs are booked here, not in the cache manager."""

    def __init__(self, cache: CacheManager) -> None:
        self.cache = cache
        self.free = list(cache.num_free_pages)
        self.slots = cache.slots.num_free

    def _take(self, need: list[int]) -> bool:
        if any(n > f for n, f in zip(need, self.free)):
            return False
        self.free = [f - n for n, f in zip(need, self.free)]
        return True

    def extend(self, seq: Sequence, computed: int, target: int) -> bool:
        need = self.cache.missing_pages(seq.seq_id, computed, target)
        return need is None or self._take(need)

    def evict(self, seq: Sequence) -> None:
        self.free = [f + n for f, n in zip(self.free, self.cache.pages_held(seq.seq_id))]
        self.slots += 1

    def admit(self, target: int) -> bool:
        if self.slots < 1 or not self._take(self.cache.pages_for_new_request(target)):
            return False
        self.slots -= 1
        return True


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
        self.waiting: deque[Sequence] = deque()  # in order of arrival; preempted ones in front
        self.running: list[Sequence] = []  # in order of admission
        self.num_preemptions = 0

    # --- requests come and go ---------------------------------------------------------------

    @property
    def capacity_tokens(self) -> int:
        return self.cache.capacity_tokens

    def has_unfinished(self) -> bool:
        return bool(self.waiting) or bool(self.running)

    def add(self, seq: Sequence) -> None:
        """Queue a request; one that the cache could not hold even alone is refused."""
        at_most = len(seq.prompt_ids) + seq.params.max_tokens
        if at_most > self.capacity_tokens:
            raise ValueError(f"prompt + max_tokens = {at_most} tokens exceeds the KV cache "
                             f"({self.capacity_tokens} tokens)")
        seq.status = SeqStatus.WAITING
        self.waiting.append(seq)

    def finish(self, seq: Sequence, reason: str | None) -> None:
        """The request is over: it leaves its queue and its pages and slot go back at once."""
        if seq.status is SeqStatus.RUNNING:
            self.running.remove(seq)
        elif seq.status is SeqStatus.WAITING and seq in self.waiting:
            self.waiting.remove(seq)
        seq.status, seq.finish_reason = SeqStatus.FINISHED, reason
        self.cache.free(seq.seq_id)

    def abort(self, request_id: str) -> Sequence | None:
        for seq in (*self.waiting, *self.running):
            if seq.request_id == request_id:
                self.finish(seq, "abort")
                return seq
        return None

    # --- planning ---------------------------------------------------------------------------

    def _share(self, pending: int, budget: int) -> int:
        """Of ``pending`` ids, how many a request gets from ``budget`` (0: it sits this step out)."""
        if pending <= budget or self.enable_chunked_prefill:
            return min(pending, budget)
        return pending if budget == self.max_num_batched_tokens else 0

    def plan(self, lookahead: int = 0) -> StepPlan:
        """Decide the next step without changing anything.  ``lookahead``: ids every running
        request will have gained by then beyond what it holds now (1 while the device is still
        sampling this step's tokens)."""
        plan = StepPlan()
        ledger = _PageLedger(self.cache)
        budget = self.max_num_batched_tokens
        unserved = deque(self.running)
        while unserved and budget > 0:
            seq = unserved.popleft()
            count = self._share(seq.num_new_tokens + lookahead, budget)
            if count == 0:
                continue
            while not ledger.extend(seq, seq.num_computed, seq.num_computed + count):
                loser = unserved.pop() if unserved else seq
                ledger.evict(loser)
                plan.preempted.append(loser)
                if loser is seq:
                    count = 0
                    break
            if count:
                plan.grant(seq, count)
                budget -= count
        # the waiting queue as it will stand: this step's victims, oldest first, then the rest
        places = self.max_num_seqs - (len(self.running) - len(plan.preempted))
        for seq in (*reversed(plan.preempted), *self.waiting):
            if budget <= 0 or places <= 0:
                break
            count = self._share(seq.length, budget)  # (a waiting request has nothing cached)
            if count == 0 or not ledger.admit(count):
                break
            plan.admitted.append(seq)
            plan.grant(seq, count)
            budget -= count
            places -= 1
        return plan

    def plan_steady_decode(self, seqs: list[Sequence]) -> StepPlan | None:
        """If, once the tokens now being sampled have arrived, the next step is exactly ``seqs``
        with one token each (nobody waiting, preempted or at its own limit), that plan; else None."""
        if self.waiting or self.running != seqs:
            return None
        if any(s.num_new_tokens or len(s.output_ids) + 1 >= s.params.max_tokens for s in seqs):
            return None
        plan = self.plan(lookahead=1)
        return plan if plan.is_decode_of(seqs) else None

    # --- carrying a plan out ----------------------------------------------------------------

    def commit(self, plan: StepPlan) -> None:
        """Apply ``plan`` (drawn up against the present state): evict, admit, take pages."""
        for seq in plan.preempted:
            self.cache.free(seq.seq_id)
            self.running.remove(seq)
            seq.forget_cache()
            self.waiting.appendleft(seq)
        self.num_preemptions += len(plan.preempted)
        for seq in plan.admitted:
            head = self.waiting.popleft()
            assert head is seq, "admission must follow the waiting queue's order"
            self.cache.add_request(seq.seq_id)
            seq.status = SeqStatus.RUNNING
            self.running.append(seq)
        for seq, count in zip(plan.seqs, plan.num_tokens):
            if self.cache.missing_pages(seq.seq_id, seq.num_computed, seq.num_computed + count):
                self.cache.grow(seq.seq_id, seq.num_computed, seq.num_computed + count)

    def schedule(self) -> StepPlan | None:
        """Plan the next step and commit it.  None if nobody gets a token (evictions that the
        plan holds are still carried out)."""
        plan = self.plan()
        self.commit(plan)
        return plan if plan.seqs else None
