"""Trace replay: feed given token ids through the model step by step and hand back logits.

Nothing is sampled.  The session drives the engine's own model, step function, cache
manager and kernels; it only keeps, per request, how many tokens have been fed.  The
reference has no such program; its nearest relatives are tests/test_engine.py:53-68 and
bench/batch_invariance.py.

A step is ``{"step": k, "entries": [{"id", "tokens", "want"}], "end": [ids]}``: every entry
brings a request's next tokens (a whole prompt, a portion cut anywhere, or one token) and
the places among them whose logits are wanted; ``end`` lists the requests that are over
after the step, whose pages and state slot go back to the pools.
"""

from __future__ import annotations

from pathlib import Path
from typing import Any

from .batch import StepEntry
from .loading import load_model
from .runner import make_runner

LIVE_REQUESTS = 8  # state slots; a trace keeps at most four requests alive


class ReplaySession:
    def __init__(self, model_dir: str | Path, dtype: str, max_tokens: int, device="cuda",
                 ops=None, page_size: int = 16) -> None:
        if ops is None:
            from ..kernels import get_ops

            ops = get_ops(device)
        self.ops, self.device, self.page_size = ops, device, page_size
        # The pool holds `max_tokens` tokens, each request's count rounded up to a multiple
        # of 64 by the caller; pages are smaller than 64, so this many pages always suffice.
        num_pages = max(-(-int(max_tokens) // page_size), 1)
        capacity = num_pages * page_size
        self.model, _ = load_model(model_dir, dtype, device, max_positions=capacity)
        spec = self.model.spec
        self.runner = make_runner(self.model, ops, device, page_size, num_pages,
                                  max_requests=LIVE_REQUESTS, max_tokens_per_step=64)
        self.cache = self.runner.cache
        self.vocab_size = spec.vocab_size
        self.fed: dict[Any, int] = {}

    def run_step(self, step: dict[str, Any]):
        """Run one step; return the ``[wanted, vocab]`` 32-bit logits (a CPU tensor) or None."""
        entries = []
        for e in step.get("entries", []):
            rid, tokens = e["id"], [int(t) for t in e["tokens"]]
            if not tokens:
                raise ValueError(f"step {step.get('step')}: request {rid!r} brings no tokens")
            if rid not in self.fed:
                self.cache.add_request(rid)
                self.fed[rid] = 0
            start = self.fed[rid]
            self.cache.grow(rid, start, start + len(tokens))
            entries.append(StepEntry(rid, tokens, start, [int(w) for w in e.get("want", [])]))
        logits = None
        if entries:
            out = self.runner.step(entries)
            if out is not None:
                logits = out.float().cpu()
            self.ops.check_errors()
            for e in entries:
                self.fed[e.req_id] += len(e.tokens)
                self.cache.release_behind_window(e.req_id, self.fed[e.req_id])
        for rid in step.get("end", []):
            if rid in self.fed:
                self.cache.free(rid)
                del self.fed[rid]
        return logits


def main(argv: list[str] | None = None) -> int:
    """The replay program: ``bin/trace_run`` and ``engine replay`` both end up here.

        trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

    Steps are read from standard input, one JSON object a line.  For a step in which something
    is wanted, ``DIR/<step>.f32`` receives the logits at the wanted places, in the order of the
    entries and of ``want``, as little-endian 32-bit floats ``[wanted, vocab]``.  After every
    step a line ``done <step>`` is printed and flushed.
    """
    import argparse
    import json
    import os
    import sys

    ap = argparse.ArgumentParser(prog="trace_run", description=main.__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (sizes the cache pool)")
    ap.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    args = ap.parse_args(argv)

    print("[trace_run] loading the model; kernels are compiled at the first call ...",
          file=sys.stderr, flush=True)
    session = ReplaySession(args.model, args.dtype, args.max_tokens, device="cuda",
                            page_size=args.block_size)
    os.makedirs(args.out, exist_ok=True)
    print("[trace_run] ready", file=sys.stderr, flush=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        logits = session.run_step(step)
        if logits is not None:
            with open(os.path.join(args.out, f"{step['step']}.f32"), "wb") as f:
                f.write(logits.contiguous().numpy().astype("<f4", copy=False).tobytes())
        print(f"done {step['step']}", flush=True)
    return 0
