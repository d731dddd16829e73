"""What the engine keeps about one request while it lives.

A request is a prompt plus the tokens produced so far.  ``num_computed`` of those ids have
their keys and values (or state) in the cache; a step feeds the ids that follow, and a token
is sampled only when a step reaches the end of the ids.  A preempted request forgets what it
computed but keeps what it produced: it is prefilled again over both (recompute preemption,
engine/runtime/scheduler.py:48-58,210-216 of the reference).  No torch here.
"""

from __future__ import annotations

import enum
from typing import Any

from ..sampling.params import SamplingParams


class SeqStatus(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


class Sequence:
    __slots__ = ("seq_id", "request_id", "prompt_ids", "params", "output_ids", "num_computed",
                 "status", "finish_reason", "num_preemptions", "seed", "processor")

    def __init__(self, seq_id: int, request_id: str, prompt_ids: list[int],
                 params: SamplingParams) -> None:
        self.seq_id = seq_id  # the key under which the cache manager knows the request
        self.request_id = request_id  # the caller's name for it
        self.prompt_ids = prompt_ids
        self.params = params
        self.output_ids: list[int] = []
        self.num_computed = 0
        self.status = SeqStatus.WAITING
        self.finish_reason: str | None = None
        self.num_preemptions = 0
        self.seed = 0  # its sampling seed: its own, or drawn when it was added
        self.processor: Any = None  # turns sampled ids into text pieces and stop decisions

    def __repr__(self) -> str:
        return (f"Sequence({self.request_id!r}, {len(self.prompt_ids)}+{len(self.output_ids)} ids, "
                f"{self.num_computed} computed, {self.status.value})")

    @property
    def all_ids(self) -> list[int]:
        return self.prompt_ids + self.output_ids

    @property
    def length(self) -> int:
        return len(self.prompt_ids) + len(self.output_ids)

    @property
    def num_new_tokens(self) -> int:
        """Ids that no step has fed yet."""
        return self.length - self.num_computed

    @property
    def decoding(self) -> bool:
        """Everything but the last produced token is in the cache."""
        return bool(self.output_ids) and self.num_computed == self.length - 1

    def ids_from(self, start: int, count: int) -> list[int]:
        """``count`` ids starting at position ``start`` of prompt + produced tokens."""
        n_prompt = len(self.prompt_ids)
        if start >= n_prompt:
            return self.output_ids[start - n_prompt: start - n_prompt + count]
        if start + count <= n_prompt:
            return self.prompt_ids[start: start + count]
        return self.prompt_ids[start:] + self.output_ids[: start + count - n_prompt]

    def forget_cache(self) -> None:
        """Preempted: nothing of it is cached any more."""
        self.num_computed = 0
        self.num_preemptions += 1
        self.status = SeqStatus.WAITING
