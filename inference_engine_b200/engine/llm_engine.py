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

import dataclasses
import itertools
import os
import random
import time
from collections import deque
from typing import Any

from ..cache.manager import CacheManager
from ..cache.storage import CacheStorage, pages_that_fit
from ..config.engine_config import EngineConfig
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .batch import StepEntry
from .graphs import DecodeGraphs, MixedGraphs
from .model import Model
from .output import OutputProcessor, RequestOutput
from .runner import ModelRunner
from .request import Sequence
from .scheduler import Scheduler


class LLMEngine:
    def __init__(self, model: Model, tokenizer: Any = None, stop_token_ids: tuple[int, ...] = (),
                 config: EngineConfig | None = None, *, ops=None, **settings) -> None:
        """``config``: the engine's settings; or give them by name (``num_blocks``,
        ``block_size``, ``max_num_seqs``, ``max_num_batched_tokens``, ``gpu_memory_utilization``,
        ``enable_chunked_prefill``, ``enable_cuda_graphs``, ``enable_mixed_graphs``, ``max_model_len``,
        ``debug_checks``: the reference's argument names, engine/runtime/engine.py:47-66) and
        they are checked as an :class:`EngineConfig`."""
        import torch

        if config is None:
            config = EngineConfig(dtype=model.env.dtype, **settings)
        elif settings:
            config = dataclasses.replace(config, **settings)
        if config.dtype != model.env.dtype:
            raise ValueError(f"the model was built for {model.env.dtype}, the engine configuration says {config.dtype}")
        self.config = config
        self.model, self.tokenizer = model, tokenizer
        self.stop_token_ids = tuple(stop_token_ids)
        self.device = model.env.device
        self.dtype = model.env.dtype
        if ops is None:
            from ..kernels import get_ops

            ops = get_ops(self.device)
        self.ops = ops
        block_size, max_num_seqs = config.block_size, config.max_num_seqs
        num_blocks = config.num_blocks
        if num_blocks is None:
            num_blocks = pages_that_fit(model.paged_groups, block_size, 2 if self.dtype == "bfloat16" else 4,
                                        self.device, config.gpu_memory_utilization)
        self.max_model_len = min(config.max_model_len or model.spec.max_position_embeddings,
                                 num_blocks * block_size if model.paged_groups else 2**62,
                                 model.env.max_positions)
        table_width = -(-self.max_model_len // block_size)
        self.cache = CacheManager(model.paged_groups, model.state_groups, num_blocks, block_size,
                                  max_num_seqs, max_pages_per_request=table_width)
        self.storage = CacheStorage(self.cache, model.env.torch_dtype, self.device)
        self.runner = ModelRunner(model, self.cache, self.storage, ops, self.device,
                                  config.max_num_batched_tokens, max_num_seqs)
        self.scheduler = Scheduler(self.cache, max_num_seqs, config.max_num_batched_tokens,
                                   config.enable_chunked_prefill)
        self.sampler = Sampler(ops, self.device, model.spec.vocab_size)
        use_graphs = config.enable_cuda_graphs
        if use_graphs is None:  # where they can be captured: on a GPU, no per-request state slots
            use_graphs = (str(self.device).startswith("cuda") and torch.cuda.is_available()
                          and not model.state_groups)
        self.graphs = DecodeGraphs(self.runner, max_num_seqs, table_width) if use_graphs else None
        use_mixed = config.enable_mixed_graphs
        if use_mixed is None:
            use_mixed = self.graphs is not None
        if use_mixed and self.graphs is None:
            raise ValueError("enable_mixed_graphs needs enable_cuda_graphs")
        self.mixed_graphs = MixedGraphs(self.graphs, config.max_num_batched_tokens) if use_mixed else None
        self.debug_checks = config.debug_checks
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
    def from_model_dir(cls, model_dir, dtype: str | None = None, device="cuda",
                       config: EngineConfig | None = None, **settings) -> "LLMEngine":
        """Load ``config.json`` and the safetensors weights of ``model_dir`` and build the
        engine; stop ids come from the folder (config and generation config)."""
        from ..config.model_config import load_stop_token_ids
        from .loading import load_model

        tokenizer = settings.pop("tokenizer", None)
        stop_ids = settings.pop("stop_token_ids", None)
        config = cls._settings(config, dtype, settings)
        model, _ = load_model(model_dir, config.dtype, device, max_positions=config.max_model_len)
        if stop_ids is None:
            stop_ids = load_stop_token_ids(model_dir)
        return cls(model, tokenizer, stop_ids, config, ops=settings.pop("ops", None))

    @classmethod
    def from_random(cls, model_config: dict, seed: int = 0, dtype: str | None = None, device="cuda",
                    config: EngineConfig | None = None, **settings) -> "LLMEngine":
        """An engine around a model of the given ``config.json`` dictionary with seeded random
        weights."""
        from .loading import random_model

        tokenizer = settings.pop("tokenizer", None)
        stop_ids = settings.pop("stop_token_ids", ())
        ops = settings.pop("ops", None)
        config = cls._settings(config, dtype, settings)
        model, _ = random_model(model_config, seed, config.dtype, device, max_positions=config.max_model_len)
        return cls(model, tokenizer, stop_ids, config, ops=ops)

    @staticmethod
    def _settings(config: EngineConfig | None, dtype: str | None, settings: dict) -> EngineConfig:
        names = {f.name for f in dataclasses.fields(EngineConfig)}
        given = {k: settings.pop(k) for k in list(settings) if k in names}
        if dtype is not None:
            given["dtype"] = dtype
        unknown = set(settings) - {"ops"}
        if unknown:
            raise TypeError(f"unknown engine settings: {sorted(unknown)}")
        return dataclasses.replace(config, **given) if config is not None else EngineConfig(**given)

    # --- requests ---------------------------------------------------------------------------

    def add_request(self, request_id: str, prompt_ids: list[int], params: SamplingParams) -> None:
        """Queue a request.  Refused with a ValueError: an id that is still live, an empty
        prompt, ids outside the vocabulary, and a request that could outgrow ``max_model_len``
        or the cache even alone (the reference's checks, engine/runtime/engine.py:144-159)."""
        problem = self._why_not(request_id, prompt_ids, params)
        if problem:
            raise ValueError(problem)
        seq = Sequence(next(self._seq_ids), request_id, list(prompt_ids), params)
        seq.seed = self._rng.getrandbits(62) if params.seed is None else params.seed
        seq.processor = OutputProcessor(self.tokenizer, params, self.stop_token_ids)
        self.scheduler.add(seq)  # (refuses what the cache could never hold)
        self._requests[request_id] = seq

    def _why_not(self, request_id: str, prompt_ids: list[int], params: SamplingParams) -> str | None:
        vocab = self.model.spec.vocab_size
        longest = len(prompt_ids) + params.max_tokens
        if request_id in self._requests:
            return f"duplicate request id {request_id!r}"
        if len(prompt_ids) == 0:
            return "prompt must have at least one token"
        if longest > self.max_model_len:
            return f"prompt + max_tokens = {longest} tokens exceeds max_model_len ({self.max_model_len})"
        if min(prompt_ids) < 0 or max(prompt_ids) >= vocab:
            return f"prompt holds a token id outside the vocabulary (0..{vocab - 1})"
        return None

    def abort(self, request_id: str) -> bool:
        """Stop a request and give its pages back now.  False if it was already done."""
        self._requests.pop(request_id, None)
        found = self.scheduler.abort(request_id) is not None
        if self._ahead is not None and not self._anyone_left(self._ahead[0]):
            self._ahead = None  # the step that is running ahead has nobody to deliver to
        return found

    def _alive(self, seq: Sequence) -> bool:
        return self._requests.get(seq.request_id) is seq

    def _anyone_left(self, seqs: list[Sequence]) -> bool:
        return any(self._alive(s) for s in seqs)

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished()

    @property
    def num_free_blocks(self) -> list[int]:
        return self.cache.num_free_pages

    # --- one step ---------------------------------------------------------------------------

    def step(self) -> list[RequestOutput]:
        started = time.perf_counter()
        preempted_before = self.scheduler.num_preemptions
        logits = kernel_times = None
        captured_mixed = False  # the step held prompt portions and ran as a captured launch sequence
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
                tokens = seq.ids_from(start, n)
                decode_tokens += n == 1 and start >= len(seq.prompt_ids)
                if not seq.output_ids and start == 0:
                    self.prompt_tokens_total += len(seq.prompt_ids)
                last = start + n == seq.length
                entries.append(StepEntry(seq.seq_id, tokens, start, [n - 1] if last else []))
                if last:
                    sampled.append(seq)
            used_graph = False
            if self.graphs is not None and len(sampled) == len(entries) and self.graphs.can_run(entries):
                logits = self.graphs.run(entries)
                used_graph = True
            elif (self.mixed_graphs is not None and not self.config.profile_kernels
                  and self.mixed_graphs.can_run(entries)):
                logits = self.mixed_graphs.run(entries)
                captured_mixed = True
            elif self.config.profile_kernels and hasattr(self.ops, "timed"):
                # (the lead: about what the host needs to launch a layer's ten or so kernels, per layer)
                with self.ops.timed(lead_ms=0.2 * len(self.model.spec.schedule)) as timer:
                    logits = self.runner.step(entries)
                kernel_times = {k: round(v["ms"], 4) for k, v in timer.summary().items()}
            else:
                logits = self.runner.step(entries)

        for seq, n in zip(seqs, counts):
            if n and self._alive(seq):  # (one that ended while this step ran ahead holds nothing)
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
            if (used_graph or captured_mixed) and len(sampled) == len(seqs):
                # while the device is busy: start the next step on the tokens it is sampling,
                # or at least pack that step's index data
                self._ahead = self._launch_ahead(seqs, pending)
                if self._ahead is None:
                    self._prepared = self._prepare_next(seqs)
            tokens, logprobs = self.sampler.collect(pending)
            for row, (seq, token) in enumerate(zip(sampled, tokens)):
                if not self._alive(seq):
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
            if self._ahead is not None and not self._anyone_left(self._ahead[0]):
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
        if kernel_times is not None:  # device ms per kind of kernel (EngineConfig.profile_kernels)
            self.step_log[-1]["kernels_ms"] = kernel_times
        return outputs

    # While the device runs a decode step the host already knows what the next one looks like
    # if nothing else happens (same requests, one position further, tokens = what is being
    # sampled now): it packs that step's index data ahead of time.  If a request finishes, is
    # aborted or preempted, or a new one arrives, the packed step is dropped and the scheduler
    # decides as usual.

    def _prepare_next(self, seqs: list[Sequence]):
        if self.graphs is None:
            return None
        # the scheduler's own answer to "what would the next step be": these requests, one
        # token each, or something else (someone waits, ends at its limit, pages run out)
        plan = self.scheduler.plan_steady_decode(seqs)
        if plan is None:
            return None
        self.scheduler.commit(plan)  # takes the pages the sampled tokens will need
        positions = [s.num_computed for s in seqs]  # where the tokens sampled now will go
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

    def warm_up(self, max_tokens: int | None = None) -> int:
        """Capture the launch sequences ahead of the first request, as the reference does when the
        engine is built (engine/runtime/cuda_graphs.py:47, 159): one decode step per batch bucket
        and one step with a prompt portion per token bucket up to ``max_tokens``, for short
        contexts of one length (captures for longer block tables, and for the other ways the decode
        attention deals contexts of very different lengths, are made when a step first needs one).  Uses
        requests of its own on an idle engine and gives their pages back.  Returns how many
        launch sequences are captured afterwards; 0 without captured steps."""
        if self.graphs is None:
            return 0
        if self.has_unfinished():
            raise RuntimeError("warm_up() wants an idle engine")
        from .batch import StepEntry

        cache, ps = self.cache, self.cache.page_size

        def run(lengths, step) -> None:
            ids = [("warm-up", i) for i in range(len(lengths))]
            held = []
            try:
                for rid, n in zip(ids, lengths):
                    cache.add_request(rid)
                    held.append(rid)
                    cache.grow(rid, 0, n)
                step([StepEntry(rid, [0] * n, 0, [n - 1]) for rid, n in zip(ids, lengths)])
            finally:
                for rid in held:
                    cache.free(rid)

        # (twice, the largest first: a capture holds the addresses of the step's buffers, and a buffer
        # that has to grow for a later step makes the earlier captures stale; the second round finds
        # every buffer as large as these steps need it and captures again what the first lost)
        free_pages = min(cache.num_free_pages)
        for _ in range(2):
            if self.mixed_graphs is not None:
                limit = min(max_tokens or self.config.max_num_batched_tokens, free_pages * ps)
                for tokens in sorted(self.mixed_graphs.token_buckets, reverse=True):
                    if 2 <= tokens <= limit:
                        run([tokens], self.mixed_graphs.run)
            for bucket in sorted(self.graphs.buckets, reverse=True):
                if bucket <= min(free_pages, cache.max_requests):
                    run([1] * bucket, self.graphs.run)
        self.ops.check_errors()
        return len(self.graphs._graphs) + (len(self.mixed_graphs._graphs) if self.mixed_graphs else 0)

    def generate(self, prompts: dict[str, list[int]], params: SamplingParams) -> dict[str, list[int]]:
        """Run ``prompts`` (request id -> token ids) to their end with the same ``params``;
        returns the produced ids per request."""
        produced: dict[str, list[int]] = {}
        for request_id, prompt in prompts.items():
            self.add_request(request_id, prompt, params)
            produced[request_id] = []
        while self.has_unfinished():
            for out in self.step():
                produced[out.request_id].append(out.token_id)
        return produced

    def snapshot(self) -> dict:
        """The engine's state as plain data, for a status page or a log: settings, totals since
        start, who runs and who waits, and the latest step records (what the reference's
        ``snapshot`` reports, engine/runtime/engine.py:300-375)."""
        sched = self.scheduler
        fields = (("id", lambda s: s.seq_id), ("request", lambda s: s.request_id),
                  ("prompt", lambda s: len(s.prompt_ids)), ("output", lambda s: len(s.output_ids)),
                  ("computed", lambda s: s.num_computed), ("max_tokens", lambda s: s.params.max_tokens),
                  ("preemptions", lambda s: s.num_preemptions))
        rows = lambda seqs: [{name: get(s) for name, get in fields} for s in seqs]  # noqa: E731
        settings = {
            "dtype": self.dtype, "block_size": self.cache.page_size,
            "num_blocks": [pool.num_pages for pool in self.cache.pools],
            "capacity_tokens": sched.capacity_tokens, "max_model_len": self.max_model_len,
            "max_num_seqs": sched.max_num_seqs,
            "max_num_batched_tokens": sched.max_num_batched_tokens,
            "cuda_graphs": self.graphs is not None, "chunked_prefill": sched.enable_chunked_prefill,
        }
        totals = {
            "steps": self.steps_total, "generated_tokens": self.generated_total,
            "finished_requests": self.finished_total, "prompt_tokens": self.prompt_tokens_total,
            "preemptions": sched.num_preemptions, "free_blocks": self.cache.num_free_pages,
        }
        return {"uptime_s": round(time.time() - self.started_at, 1), "config": settings,
                "totals": totals, "running": rows(sched.running),
                "waiting": rows(itertools.islice(sched.waiting, 32)), "num_waiting": len(sched.waiting),
                "steps": list(self.step_log)[-120:]}
