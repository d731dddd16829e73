"""How one request wants its tokens chosen and when it stops.

The field names, their defaults and their allowed ranges are the reference's request schema
(engine/runtime/params.py:8-41), so that a caller of the reference finds the same knobs; the
checks are written as a table of ranges.  No torch.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

# field -> (lowest, lowest allowed itself?, highest, highest allowed itself?, how the message says it)
_RANGES = {
    "temperature": (0.0, True, math.inf, False, ">= 0"),
    "top_k": (0, True, math.inf, False, ">= 0"),
    "top_p": (0.0, False, 1.0, True, "in (0, 1]"),
    "min_p": (0.0, True, 1.0, False, "in [0, 1)"),
    "repetition_penalty": (0.0, False, math.inf, False, "> 0"),
    "max_tokens": (1, True, math.inf, False, ">= 1"),
    "top_logprobs": (0, True, 20, True, "in [0, 20]"),
}


@dataclass(frozen=True)
class SamplingParams:
    """``temperature`` 0 takes the most likely token; ``top_k`` 0, ``top_p`` 1 and ``min_p`` 0
    cut nothing off; ``repetition_penalty`` 1 changes nothing; ``seed`` makes a request's draws
    repeatable whatever else is in the batch; ``stop`` strings need a tokenizer;
    ``logprobs`` reports the chosen token's log-probability and ``top_logprobs`` that of up to
    20 most likely alternatives."""

    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    max_tokens: int = 256
    seed: int | None = None
    stop: tuple[str, ...] = ()
    logprobs: bool = False
    top_logprobs: int = 0

    def __post_init__(self) -> None:
        for name, (low, low_ok, high, high_ok, wording) in _RANGES.items():
            value = getattr(self, name)
            above = value >= low if low_ok else value > low
            below = value <= high if high_ok else value < high
            if not (above and below):  # (also catches NaN)
                raise ValueError(f"{name} must be {wording}, not {value!r}")
        if self.top_logprobs and not self.logprobs:
            raise ValueError("top_logprobs needs logprobs=True")
        if isinstance(self.stop, str):
            object.__setattr__(self, "stop", (self.stop,))
        elif not isinstance(self.stop, tuple):
            object.__setattr__(self, "stop", tuple(self.stop))

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0
