"""Per-request output handling: stop ids, stop strings and ``max_tokens``
(engine/runtime/stop.py:12-72), and the record a step returns for each new token
(engine/runtime/engine.py:31-43)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from ..sampling.params import SamplingParams


@dataclass
class RequestOutput:
    request_id: str
    token_id: int
    text: str  # detokenised delta, "" without a tokenizer
    finished: bool
    finish_reason: str | None  # "stop" | "length" | "abort"
    prompt_tokens: int
    completion_tokens: int
    logprob: float | None = None
    top_logprobs: list[tuple[int, float]] | None = None


class OutputProcessor:
    """A stop id ends the request with reason "stop" and is still its last token; reaching
    ``max_tokens`` ends it with "length".  Stop strings need a tokenizer: the text produced so
    far is decoded again after every token, and what could still become a stop string is held
    back."""

    def __init__(self, tokenizer: Any, params: SamplingParams, stop_token_ids) -> None:
        if params.stop and tokenizer is None:
            raise ValueError("stop strings need a tokenizer; without one use stop token ids")
        self.tokenizer, self.params = tokenizer, params
        self.stop_ids = set(stop_token_ids)
        self.ids: list[int] = []
        self.emitted = 0
        self.holdback = max((len(s) for s in params.stop), default=1) - 1

    def process(self, token_id: int) -> tuple[str, bool, str | None]:
        self.ids.append(token_id)
        if token_id in self.stop_ids:
            return self._flush(self._text(self.ids[:-1])), True, "stop"
        text = self._text(self.ids)
        if text.endswith("�"):  # an unfinished multi-byte character: wait for the rest
            text = text[: self.emitted] if len(text) > self.emitted else text
        hits = [i for s in self.params.stop if (i := text.find(s, max(self.emitted - len(s), 0))) != -1]
        if hits:
            return self._emit(text, min(hits)), True, "stop"
        if len(self.ids) >= self.params.max_tokens:
            return self._flush(text), True, "length"
        return self._emit(text, len(text) - self.holdback), False, None

    def _text(self, ids: list[int]) -> str:
        if self.tokenizer is None or not ids:
            return ""
        return self.tokenizer.decode(ids, skip_special_tokens=True)

    def _emit(self, text: str, end: int) -> str:
        if end <= self.emitted:
            return ""
        out, self.emitted = text[self.emitted:end], end
        return out

    def _flush(self, text: str) -> str:
        return self._emit(text, len(text))
