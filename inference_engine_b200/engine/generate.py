"""The Python entry point for plain generation, in the reference's manner
(engine/runtime/generate.py:26-90): prompts as lists of token ids in, one ``StepOutput`` per
sequence and step out, until every sequence has finished.  The reference runs a static,
left-padded batch over a contiguous cache there; here the same call drives the paged engine
(continuous batching, chunked prefill), so there is one path from ids to ids."""

from __future__ import annotations

from collections.abc import Iterator
from dataclasses import dataclass
from typing import Any

from ..sampling.params import SamplingParams
from .llm_engine import LLMEngine


@dataclass
class StepOutput:
    seq_index: int  # which prompt of the batch
    token_id: int
    text: str  # detokenised delta, "" without a tokenizer
    finished: bool
    finish_reason: str | None = None  # "stop" | "length"


def generate(model: Any, tokenizer: Any, prompts: list[list[int]], params: SamplingParams,
             stop_token_ids: tuple[int, ...] = (), **engine_kwargs) -> Iterator[StepOutput]:
    """``model``: a loaded :class:`~inference_engine_b200.engine.model.Model` or an
    :class:`LLMEngine` to reuse.  A stop token is yielded as the sequence's last token."""
    if not prompts or any(len(p) == 0 for p in prompts):
        raise ValueError("every prompt needs at least one token")
    if isinstance(model, LLMEngine):
        engine = model
    else:
        longest = max(len(p) for p in prompts) + params.max_tokens
        block_size = engine_kwargs.get("block_size", 16)
        engine_kwargs.setdefault("num_blocks", len(prompts) * (-(-longest // block_size) + 1))
        engine_kwargs.setdefault("max_num_seqs", max(len(prompts), 1))
        engine_kwargs.setdefault("max_num_batched_tokens", max(2048, len(prompts)))
        engine = LLMEngine(model, tokenizer, stop_token_ids, **engine_kwargs)
    index = {}
    for i, prompt in enumerate(prompts):
        rid = f"generate-{id(prompts)}-{i}"
        index[rid] = i
        engine.add_request(rid, prompt, params)
    while any(rid in engine._requests for rid in index):
        for out in engine.step():
            if out.request_id in index:
                yield StepOutput(index[out.request_id], out.token_id, out.text, out.finished,
                                 out.finish_reason)
