"""The engine: requests in, tokens out, one step at a time.

    engine = LLMEngine.from_model_dir("path/to/model", dtype="bfloat16")
    engine.add_request("r1", prompt_ids, SamplingParams(max_tokens=64))
    while engine.has_unfinished():
        for out in engine.step():
            print(out.request_id, out.token_id)

The public surface is the reference's ``LLMEngine`` (engine/runtime/engine.py:46-387):
``add_request``, ``step``, ``generate``, ``abort``, ``has_unfinished``, ``snapshot``, with the
same argument names where they apply.  Token ids go in and come out; a tokenizer is optional
and only used for text deltas and stop strings.  Not thread-safe.
"""

from __future__ import annotations

import itertools
import os
import random
import time
from collections import deque
from typing import Any

from ..cache.manager import CacheManager
from ..cache.storage import CacheStorage
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .batch import StepEntry
from .graphs import DecodeGraphs
from .model import Model
from .output import OutputProcessor, RequestOutput
from .runner import ModelRunner
from .scheduler import Scheduler, Sequence


class LLMEngine:
    def __init__(self, model: Model, tokenizer: Any = None, stop_token_ids: tuple[int, ...] = (), *,
                 num_blocks: int | None = None, block_size: int = 16, max_num_seqs: int = 64,
                 max_num_batched_tokens: int = 4096, gpu_memory_utilization: float = 0.9,
                 enable_chunked_prefill: bool = True, enable_cuda_graphs: bool | None = None,
                 max_model_len: int | None = None, debug_checks: bool = False, ops=None) -> None:
        import torch

        self.model, self.tokenizer = model, tokenizer
        self.stop_token_ids = tuple(stop_token_ids)
        self.device = model.env.device
        self.dtype = model.env.dtype
        if ops is None:
            from ..kernels import get_ops

            ops = get_ops(self.device)
        self.ops = ops
        elt = 2 if self.dtype == "bfloat16" else 4
        if num_blocks is None:
            num_blocks = self._blocks_that_fit(block_size, gpu_memory_utilization, elt)
        self.max_model_len = min(max_model_len or model.spec.max_position_embeddings,
                                 num_blocks * block_size if model.paged_groups else 2**62,
                                 model.env.max_positions)
        self.cache = CacheManager(model.paged_groups, model.state_groups, num_blocks, block_size,
                                  max_num_seqs, max_pages_per_request=-(-self.max_model_len // block_size))
        self.storage = CacheStorage(self.cache, model.env.torch_dtype, self.device)
        self.runner = ModelRunner(model, self.cache, self.storage, ops, self.device,
                                  max_num_batched_tokens, max_num_seqs)
        self.scheduler = Scheduler(self.cache, max_num_seqs, max_num_batched_tokens,
                                   enable_chunked_prefill)
        self.sampler = Sampler(ops, self.device, model.spec.vocab_size)
        on_cuda = str(self.device).startswith("cuda") and torch.cuda.is_available()
        if enable_cuda_graphs is None:
            enable_cuda_graphs = on_cuda and not model.state_groups
        self.graphs = None
        if enable_cuda_graphs:
            self.graphs = DecodeGraphs(self.runner, max_num_seqs, -(-self.max_model_len // block_size))
        self.debug_checks = debug_checks
        self._seq_ids = itertools.count()
        self._requests: dict[str, Sequence] = {}
        self._rng = random.Random()
        self._prepared = None
        self._ahead = None  # a decode step launched before the previous step's tokens were fetched
        self.launch_ahead = os.environ.get("IE_B200_LAUNCH_AHEAD", "1") != "0"
        self.step_log: deque[dict] = deque(maxlen=240)
        self.steps_total = self.generated_total = self.finished_total = 0
        self.prompt_tokens_total = 0
        self.started_at = time.time()

    # --- construction helpers ---------------------------------------------------------------

    @classmethod
    def from_model_dir(cls, model_dir, dtype: str = "bfloat16", device="cuda",
                       max_model_len: int | None = None, **kwargs) -> "LLMEngine":
        """Load ``config.json`` and the safetensors weights of ``model_dir`` and build the
        engine; stop ids come from the folder (config and generation config)."""
        from ..config.model_config import load_stop_token_ids
        from .loading import load_model

        model, cfg = load_model(model_dir, dtype, device, max_positions=max_model_len)
        kwargs.setdefault("stop_token_ids", load_stop_token_ids(model_dir))
        return cls(model, max_model_len=max_model_len, **kwargs)

    @classmethod
    def from_random(cls, config: dict, seed: int = 0, dtype: str = "bfloat16", device="cuda",
                    max_model_len: int | None = None, **kwargs) -> "LLMEngine":
        from .loading import random_model

        model, cfg = random_model(config, seed, dtype, device, max_positions=max_model_len)
        return cls(model, max_model_len=max_model_len, **kwargs)

    def _blocks_that_fit(self, block_size: int, utilization: float, elt: int) -> int:
        """(free - (1 - utilization) * total - 512 MiB) // bytes per page over all groups
        (engine/runtime/engine.py:130-140)."""
        import torch

        if not str(self.device).startswith("cuda"):
            raise ValueError("pass num_blocks explicitly when not running on CUDA")
        free, total = torch.cuda.mem_get_info(self.device)
        budget = free - (1 - utilization) * total - 512 * 2**20
        per_page = sum(g.bytes_per_page(block_size, elt) for g in self.model.paged_groups) or 1
        blocks = int(budget // per_page)
        if blocks < 1:
            raise RuntimeError("no GPU memory left for the KV cache")
        return blocks

    # --- requests ---------------------------------------------------------------------------

    def add_request(self, request_id: str, prompt_ids: list[int], params: SamplingParams) -> None:
        if request_id in self._requests:
            raise ValueError(f"duplicate request id {request_id!r}")
        if not prompt_ids:
            raise ValueError("prompt must have at least one token")
        if len(prompt_ids) + params.max_tokens > self.max_model_len:
            raise ValueError(f"prompt + max_tokens = {len(prompt_ids) + params.max_tokens} tokens "
                             f"exceeds max_model_len ({self.max_model_len})")
        vocab = self.model.spec.vocab_size
        if any(not 0 <= t < vocab for t in prompt_ids):
            raise ValueError(f"prompt holds a token id outside the vocabulary (0..{vocab - 1})")
        seq = Sequence(next(self._seq_ids), request_id, list(prompt_ids), params)
        seq.seed = params.seed if params.seed is not None else self._rng.getrandbits(62)
        seq.processor = OutputProcessor(self.tokenizer, params, self.stop_token_ids)
        self.scheduler.add(seq)  # raises if it can never fit
        self._requests[request_id] = seq

    def abort(self, request_id: str) -> bool:
        """Stop a request and give its pages back now.  False if it was already done."""
        self._requests.pop(request_id, None)
        return self.scheduler.abort(request_id) is not None

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished()

    @property
    def num_free_blocks(self) -> list[int]:
        return self.cache.num_free_pages

    # --- one step ---------------------------------------------------------------------------

    def step(self) -> list[RequestOutput]:
        started = time.perf_counter()
        preempted_before = self.scheduler.num_preemptions
        logits = None
        ahead, self._ahead = self._ahead, None
        prepared, self._prepared = self._prepared, None
        if ahead is not None:
            # This step is already running on the device (see _launch_ahead).
            seqs, pending, logits = ahead
            sampled, counts, used_graph, decode_tokens = seqs, [0] * len(seqs), True, len(seqs)
        elif prepared is not None and self._prepared_still_valid(prepared):
            # Steady decoding: this step was packed while the device worked on the last one.
            seqs = prepared[0]
            logits = self.graphs.run_prepared(prepared[1], [s.output_ids[-1] for s in seqs])
        if ahead is not None:
            pass
        elif logits is not None:
            sampled, counts, used_graph = seqs, [1] * len(seqs), True
            decode_tokens = len(seqs)
        else:
            batch = self.scheduler.schedule()
            if batch is None:
                if self.scheduler.waiting and not self.scheduler.running:
                    raise RuntimeError("scheduler made no progress with an idle engine")
                return []
            seqs, counts = batch.seqs, batch.num_tokens
            entries, sampled = [], []
            decode_tokens = 0
            for seq, n in zip(seqs, counts):
                start = seq.num_computed
                n_prompt = len(seq.prompt_ids)
                if n == 1 and start >= n_prompt:
                    tokens = [seq.output_ids[start - n_prompt]]
                    decode_tokens += 1
                elif start + n <= n_prompt:
                    tokens = seq.prompt_ids[start:start + n]
                else:
                    tokens = (seq.prompt_ids + seq.output_ids)[start:start + n]
                if not seq.output_ids and start == 0:
                    self.prompt_tokens_total += n_prompt
                last = start + n == seq.length
                entries.append(StepEntry(seq.seq_id, tokens, start, [n - 1] if last else []))
                if last:
                    sampled.append(seq)
            used_graph = False
            if self.graphs is not None and len(sampled) == len(entries) and self.graphs.can_run(entries):
                logits = self.graphs.run(entries)
                used_graph = True
            else:
                logits = self.runner.step(entries)

        for seq, n in zip(seqs, counts):
            seq.num_computed += n
            self.cache.release_behind_window(seq.seq_id, seq.num_computed)

        outputs: list[RequestOutput] = []
        if sampled:
            if ahead is None:
                params = [s.params for s in sampled]
                needs_history = any(p.repetition_penalty != 1.0 for p in params)
                pending = self.sampler.launch(
                    logits, params, [s.seed for s in sampled], [len(s.output_ids) for s in sampled],
                    [s.all_ids for s in sampled] if needs_history else None,
                    history_keys=[s.seq_id for s in sampled] if needs_history else None)
            if used_graph and len(sampled) == len(seqs):
                # while the device is busy: start the next step on the tokens it is sampling,
                # or at least pack that step's index data
                self._ahead = self._launch_ahead(seqs, pending)
                if self._ahead is None:
                    self._prepared = self._prepare_next(seqs)
            tokens, logprobs = self.sampler.collect(pending)
            for row, (seq, token) in enumerate(zip(sampled, tokens)):
                if self._requests.get(seq.request_id) is not seq:
                    continue  # it ended or was aborted after this step had been launched ahead
                seq.output_ids.append(token)
                text, finished, reason = seq.processor.process(token)
                out = RequestOutput(seq.request_id, token, text, finished, reason,
                                    len(seq.prompt_ids), len(seq.output_ids))
                if seq.params.logprobs:
                    out.logprob = logprobs[row]
                    if seq.params.top_logprobs:
                        out.top_logprobs = self.sampler.top_logprobs(logits[row], seq.params.top_logprobs)
                if finished:
                    self.scheduler.finish(seq, reason)
                    self._requests.pop(seq.request_id, None)
                outputs.append(out)
            if self._ahead is not None and not any(
                    self._requests.get(s.request_id) is s for s in self._ahead[0]):
                self._ahead = None  # nobody is left to take that step's tokens
        if self.debug_checks:
            self.cache.check_invariants()
            self.ops.check_errors()
        self.steps_total += 1
        self.generated_total += len(outputs)
        self.finished_total += sum(o.finished for o in outputs)
        self.step_log.append({
            "step": self.steps_total,
            "ms": round((time.perf_counter() - started) * 1000, 3),
            "seqs": len(seqs),
            "prefill_tokens": max(sum(counts) - decode_tokens, 0),  # (a step launched ahead was counted when it was launched)
            "decode_tokens": decode_tokens,
            "graph": used_graph,
            "preempted": self.scheduler.num_preemptions - preempted_before,
        })
        return outputs

    # While the device runs a decode step the host already knows what the next one looks like
    # if nothing else happens (same requests, one position further, tokens = what is being
    # sampled now): it packs that step's index data ahead of time.  If a request finishes, is
    # aborted or preempted, or a new one arrives, the packed step is dropped and the scheduler
    # decides as usual.

    def _prepare_next(self, seqs: list[Sequence]):
        if self.graphs is None or self.scheduler.waiting or self.scheduler.running != seqs:
            return None
        positions = []
        for seq in seqs:
            pos = seq.num_computed  # where the token sampled now will go
            if len(seq.output_ids) + 1 >= seq.params.max_tokens:
                return None  # it ends with this token
            if not self.cache.try_grow(seq.seq_id, pos, pos + 1):
                return None  # pages ran out: the scheduler has to preempt
            positions.append(pos)
        handle = self.graphs.prepare([s.seq_id for s in seqs], positions)
        return (list(seqs), handle) if handle is not None else None

    # One step further: with greedy or seeded sampling that needs nothing from the host (no
    # repetition penalty, no log-probabilities) the next decode step can run on the tokens the
    # device is sampling right now.  It is launched before those tokens are fetched, so the
    # device never waits for the host between decode steps.  What the host learns too late (a
    # stop token, an abort) costs one row of that step, which is dropped; its cache page goes
    # back with the request's other pages, and everything is ordered on one stream.

    def _launch_ahead(self, seqs: list[Sequence], pending):
        if not self.launch_ahead or self.graphs is None:
            return None
        if any(s.params.repetition_penalty != 1.0 or s.params.logprobs for s in seqs):
            return None
        prepared = self._prepare_next(seqs)
        if prepared is None:
            return None
        logits = self.graphs.run_prepared(prepared[1], pending[0], count=len(seqs))
        if logits is None:
            return None
        for seq in seqs:
            seq.num_computed += 1
            self.cache.release_behind_window(seq.seq_id, seq.num_computed)
        nxt = self.sampler.launch(logits, [s.params for s in seqs], [s.seed for s in seqs],
                                  [len(s.output_ids) + 1 for s in seqs], None)
        return (list(seqs), nxt, logits)

    def _prepared_still_valid(self, prepared) -> bool:
        seqs = prepared[0]
        return (not self.scheduler.waiting and self.scheduler.running == seqs
                and all(s.num_computed == s.length - 1 for s in seqs))

    def generate(self, prompts: dict[str, list[int]], params: SamplingParams) -> dict[str, list[int]]:
        """Run requests to completion; returns the generated token ids per request."""
        for request_id, prompt in prompts.items():
            self.add_request(request_id, prompt, params)
        tokens: dict[str, list[int]] = {rid: [] for rid in prompts}
        while self.has_unfinished():
            for out in self.step():
                tokens[out.request_id].append(out.token_id)
        return tokens

    def snapshot(self) -> dict:
        """Counters and queue state as plain data (engine/runtime/engine.py:300-375)."""
        sched = self.scheduler

        def describe(seq: Sequence) -> dict:
            return {"id": seq.seq_id, "request": seq.request_id, "prompt": len(seq.prompt_ids),
                    "output": len(seq.output_ids), "computed": seq.num_computed,
                    "max_tokens": seq.params.max_tokens, "preemptions": seq.num_preemptions}

        return {
            "uptime_s": round(time.time() - self.started_at, 1),
            "config": {"dtype": self.dtype, "block_size": self.cache.page_size,
                       "num_blocks": [p.num_pages for p in self.cache.pools],
                       "capacity_tokens": sched.capacity_tokens, "max_model_len": self.max_model_len,
                       "max_num_seqs": sched.max_num_seqs,
                       "max_num_batched_tokens": sched.max_num_batched_tokens,
                       "cuda_graphs": self.graphs is not None,
                       "chunked_prefill": sched.enable_chunked_prefill},
            "running": [describe(s) for s in sched.running],
            "waiting": [describe(s) for s in list(sched.waiting)[:32]],
            "num_waiting": len(sched.waiting),
            "totals": {"steps": self.steps_total, "generated_tokens": self.generated_total,
                       "finished_requests": self.finished_total,
                       "prompt_tokens": self.prompt_tokens_total,
                       "preemptions": sched.num_preemptions,
                       "free_blocks": self.cache.num_free_pages},
            "steps": list(self.step_log)[-120:],
        }
