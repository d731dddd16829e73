#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The workload is the Llama 3.2 1B shape with seeded random weights in bfloat16 (16 layers,
hidden 2048, 32 query / 8 key-value heads of 64, feed-forward 8192, vocabulary 128256, tied
head): a batch of 8 requests with 1024-token uniform-random prompts, decoded one token per
request and step over 16-token cache pages.  A "step" is one decode step.

``value``      decoded tokens per second, timed on the device with CUDA events around K steps
               of the engine's step function (captured launch sequence, index data copied in,
               argmax included);
``e2e``        the same through ``LLMEngine.step()``: host token lists in, host tokens out,
               wall clock with a device synchronisation on both sides;
``prefill``    one 2,048-token prompt through the step function;
``roofline``   bytes the decode step has to read (every weight once, the live cache) / time;
``points``     decode tokens per second at batch 1 and 64, each with its fraction of the HBM
               roofline (``decode_b1_frac``, ``decode_b64_frac``);
``kernels``    where the time goes: CUDA-event time of every kind of kernel inside an eagerly
               launched decode step (batch 8, and the attention at batch 64) and inside the
               2,048-token prefill, per launch, with the bytes or flops it has to move and the
               fraction of the measured peak that makes.

``--impl reference`` runs the unmodified reference engine (installed under baseline/_ref) on
the same shape and batch through its own ``load_model`` / ``LLMEngine`` and prints the same
line with ``"impl": "reference"``, or an ``unavailable`` line saying why it cannot.
More than one GPU is not supported: the engine is a single-GPU engine.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LLAMA_1B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 16, "hidden_size": 2048, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192, "vocab_size": 128256,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 131072,
    "bos_token_id": 128000, "eos_token_id": [128001, 128008, 128009], "torch_dtype": "bfloat16",
}
PROMPT_LEN, PREFILL_LEN, BLOCK_SIZE, MAX_CONTEXT = 1024, 2048, 16, 8192
LEAD_MS = 2.0  # the device is kept busy this long before launches that are timed without the host's share
METRIC = "decode tokens/s, Llama 3.2 1B shape, batch 8"  # both arms print the same string


def measured_peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            raw = json.loads(path.read_text())
            flat = {}

            def walk(d):
                for k, v in d.items():
                    if isinstance(v, dict):
                        walk(v)
                    elif isinstance(v, (int, float)):
                        flat.setdefault(k, float(v))

            walk(raw)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                return flat, "measured"
        except (OSError, ValueError):
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while timed regions run."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.samples: list[list[str]] = []
        self._proc = None
        self._thread = None

    def start(self) -> None:
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self._thread = threading.Thread(target=self._read, daemon=True)
        self._thread.start()

    def _read(self) -> None:
        for line in self._proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append(parts)

    def stop(self) -> dict:
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
        mhz = [int(s[0]) for s in self.samples if s[0].isdigit()]
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i] == "Active" for s in self.samples)]
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(self.samples)}


def weight_bytes_read_per_step(cfg: dict) -> int:
    h, i = cfg["hidden_size"], cfg["intermediate_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = h * (q + 2 * kv) + q * h + 3 * h * i
    return 2 * (cfg["num_hidden_layers"] * per_layer + cfg["vocab_size"] * h)  # head = tied table


def kv_bytes_per_token(cfg: dict) -> int:
    return 2 * cfg["num_hidden_layers"] * cfg["num_key_value_heads"] * cfg["head_dim"] * 2


def prefill_flops(cfg: dict, tokens: int) -> float:
    h, i = cfg["hidden_size"], cfg["intermediate_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = h * (q + 2 * kv) + q * h + 3 * h * i
    gemm = 2.0 * tokens * cfg["num_hidden_layers"] * per_layer + 2.0 * cfg["vocab_size"] * h
    attn = cfg["num_hidden_layers"] * 2.0 * tokens * tokens * q  # causal: half of 4 T^2 nh hd
    return gemm + attn


# --- our engine ---------------------------------------------------------------------------------


def decode_device_timed(engine, batch: int, steps: int, warmup: int, seed: int, breakdown: bool = False):
    """Prefill `batch` prompts, then time `steps` decode steps of the step function on the
    device.  Returns (tokens/s, ms per step, mean context, launches of our kernels, and with
    `breakdown` the device time per kind of kernel of an eagerly launched step)."""
    import torch

    from inference_engine_b200.engine.batch import StepEntry

    runner, cache, vocab = engine.runner, engine.cache, engine.model.spec.vocab_size
    g = torch.Generator().manual_seed(seed)
    prompts = torch.randint(0, vocab, (batch, PROMPT_LEN), generator=g).tolist()
    feed = torch.randint(0, vocab, (warmup + steps + 1, batch), generator=g).tolist()
    ids = [f"bench-{seed}-{i}" for i in range(batch)]
    for rid, prompt in zip(ids, prompts):
        cache.add_request(rid)
        cache.grow(rid, 0, PROMPT_LEN)
    for start in range(0, batch, 4):  # prefill in steps of at most 4 prompts
        runner.step([StepEntry(rid, p, 0, []) for rid, p in zip(ids[start:start + 4], prompts[start:start + 4])])
    out = torch.empty(batch, dtype=torch.int32, device=engine.device)
    pos = PROMPT_LEN

    def one(k: int) -> None:
        nonlocal pos
        for rid in ids:
            cache.grow(rid, pos, pos + 1)
        entries = [StepEntry(rid, [feed[k][i]], pos, [0]) for i, rid in enumerate(ids)]
        logits = engine.graphs.run(entries) if engine.graphs is not None else runner.step(entries)
        engine.ops.argmax(logits, out)
        pos += 1

    for k in range(warmup):
        one(k)
    torch.cuda.synchronize()
    launches_before = engine.ops.launches
    start_evt, end_evt = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    first_ctx = pos + 1
    start_evt.record()
    for k in range(warmup, warmup + steps):
        one(k)
    end_evt.record()
    torch.cuda.synchronize()
    ms = start_evt.elapsed_time(end_evt)
    launches = engine.ops.launches - launches_before
    if engine.graphs is not None:
        launches += steps * engine.graphs.kernels_per_replay(batch)
    engine.ops.check_errors()
    kinds = None
    if breakdown:  # one more step, launched eagerly, and its kernels again kind by kind
        for rid in ids:
            cache.grow(rid, pos, pos + 1)
        kinds = time_kinds(engine, [StepEntry(rid, [feed[0][i]], pos, [0]) for i, rid in enumerate(ids)])
        pos += 1
    for rid in ids:
        cache.free(rid)
    mean_ctx = (first_ctx + pos) / 2
    return batch * steps / (ms / 1e3), ms / steps, mean_ctx, launches, kinds


def decode_end_to_end(engine, batch: int, steps: int, warmup: int, seed: int):
    """The same through LLMEngine.step(): host token lists in, host tokens out."""
    import torch

    from inference_engine_b200 import SamplingParams

    vocab = engine.model.spec.vocab_size
    g = torch.Generator().manual_seed(seed + 1)
    prompts = torch.randint(0, vocab, (batch, PROMPT_LEN), generator=g).tolist()
    params = SamplingParams(temperature=0.0, max_tokens=warmup + steps + 8)
    for i, p in enumerate(prompts):
        engine.add_request(f"e2e-{seed}-{i}", p, params)
    produced = 0
    while produced < batch * warmup:  # prefill and the warm-up decode steps
        produced += len(engine.step())
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    tokens = 0
    for _ in range(steps):
        tokens += len(engine.step())
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    h2d = engine.runner.last_h2d_bytes
    for i in range(batch):
        engine.abort(f"e2e-{seed}-{i}")
    return tokens / elapsed, h2d, batch * 4 + 16  # the tokens and the kernels' 16-byte error word


def prefill_timed(engine, repeats: int = 5):
    import torch

    from inference_engine_b200.engine.batch import StepEntry

    runner, cache, vocab = engine.runner, engine.cache, engine.model.spec.vocab_size
    g = torch.Generator().manual_seed(99)
    times = []
    for r in range(repeats + 2):
        prompt = torch.randint(0, vocab, (PREFILL_LEN,), generator=g).tolist()
        rid = f"prefill-{r}"
        cache.add_request(rid)
        cache.grow(rid, 0, PREFILL_LEN)
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        runner.step([StepEntry(rid, prompt, 0, [PREFILL_LEN - 1])])
        e.record()
        torch.cuda.synchronize()
        if r >= 2:
            times.append(s.elapsed_time(e))
        cache.free(rid)
    # once more, and its kernels again kind by kind
    prompt = torch.randint(0, vocab, (PREFILL_LEN,), generator=g).tolist()
    cache.add_request("prefill-kinds")
    cache.grow("prefill-kinds", 0, PREFILL_LEN)
    kinds = time_kinds(engine, [StepEntry("prefill-kinds", prompt, 0, [PREFILL_LEN - 1])])
    cache.free("prefill-kinds")
    return statistics.median(times), kinds


def time_kinds(engine, entries, passes: int = 5) -> dict:
    """Run `entries` as one eagerly launched step while the kernel set records its calls, then
    launch every kind of kernel again by itself: all of the step's launches of that kind (one per
    layer, each on its own layer's weights and cache) back to back between two CUDA events,
    queued behind a busy device so that the host's launch time is not in it, the L2 flushed
    before every pass.  Returns kind -> {"launches", "ms"} (median of `passes`)."""
    import torch

    ops = engine.ops
    with ops.recording() as calls:
        engine.runner.step(entries)
    torch.cuda.synchronize()
    by_kind: dict[str, list] = {}
    for kind, call in calls:
        by_kind.setdefault(kind, []).append(call)
    flush = torch.empty(256 * 2**20, dtype=torch.uint8, device=engine.device)
    out = {}
    for kind, launches in by_kind.items():
        times = []
        for _ in range(passes + 1):
            flush.zero_()
            ops.busy_wait(LEAD_MS)
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for call in launches:
                call()
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop))
        out[kind] = {"launches": len(launches), "ms": statistics.median(times[1:])}
    ops.check_errors()
    return out


KINDS = {"linear:attn.qkv": "K3_qkv", "attention.decode": "K5_decode_attention",
         "attention.prefill": "K6_prefill_attention", "linear:mixer.delta": "K7_out_proj",
         "linear:ffn.gate_up": "K8_gate_up", "linear:ffn.delta": "K10_down", "linear:head": "K11_head",
         "norm": "K2_norm", "rotary+cache": "K4_rotary_cache", "activation": "K9_silu_mul",
         "embedding": "K1_embedding"}


def kernel_rows(cfg: dict, kinds: dict, peaks: dict, tokens: int, batch: int, ctx: float, decode: bool) -> dict:
    """Per kind of kernel: microseconds per launch and what that is of the measured peak: of the
    copy bandwidth for the bytes a decode launch has to read (its weights once; for the attention
    the batch's cached keys and values of one layer), of the burst bf16 rate for the flops of a
    prefill launch.  Kinds without such a figure (norms, rotary, activation) give the time only."""
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    weights = {"K3_qkv": h * (q + 2 * kv), "K7_out_proj": q * h, "K8_gate_up": 2 * h * i,
               "K10_down": i * h, "K11_head": v * h}
    rows = {}
    for kind, row in kinds.items():
        name = KINDS.get(kind, kind)
        us = row["ms"] / row["launches"] * 1e3
        out = {"us": round(us, 2), "launches": row["launches"]}
        if decode and name in weights:
            gbs = 2 * weights[name] / (us * 1e-6) / 1e9
            out.update(gbs=round(gbs, 1), frac=round(gbs / peaks["hbm_gbs"], 3))
        elif decode and name == "K5_decode_attention":
            gbs = batch * ctx * 2 * kv * 2 / (us * 1e-6) / 1e9
            out.update(gbs=round(gbs, 1), frac=round(gbs / peaks["hbm_gbs"], 3))
        elif not decode and name in weights and name != "K11_head":
            tflops = 2.0 * tokens * weights[name] / (us * 1e-6) / 1e12
            out.update(tflops=round(tflops, 1), frac=round(tflops / peaks["bf16_tflops"], 3))
        elif not decode and name == "K6_prefill_attention":
            tflops = 2.0 * tokens * tokens * q / (us * 1e-6) / 1e12  # causal: half of 4 T^2 nh hd
            out.update(tflops=round(tflops, 1), frac=round(tflops / peaks["bf16_tflops"], 3))
        rows[name] = out
    return rows


def run_ours(args) -> dict:
    import torch

    from inference_engine_b200.engine.llm_engine import LLMEngine

    peaks, peaks_kind = measured_peaks()
    cfg = dict(LLAMA_1B)
    layers_run = cfg["num_hidden_layers"]
    torch.cuda.set_device(0)
    max_batch = 64
    tokens_needed = max_batch * (PROMPT_LEN + args.warmup + args.steps + 64) + 4 * PREFILL_LEN
    engine = LLMEngine.from_random(
        cfg, seed=0, dtype="bfloat16", device="cuda", max_model_len=MAX_CONTEXT,
        num_blocks=-(-tokens_needed // BLOCK_SIZE), block_size=BLOCK_SIZE, max_num_seqs=max_batch,
        max_num_batched_tokens=4 * PROMPT_LEN, enable_cuda_graphs=True)
    sampler = ClockSampler()
    sampler.start()
    tps, ms_step, mean_ctx, launches, kinds8 = decode_device_timed(engine, args.batch, args.steps, args.warmup, 1,
                                                                   breakdown=True)
    e2e_tps, h2d, d2h = decode_end_to_end(engine, args.batch, args.steps, args.warmup, 2)
    prefill_ms, kinds_prefill = prefill_timed(engine)
    small = max(args.steps // 2, 16)
    b1, ms1, ctx1, _, _ = decode_device_timed(engine, 1, small, args.warmup, 3)
    b64, ms64, ctx64, _, kinds64 = decode_device_timed(engine, 64, small, args.warmup, 4, breakdown=True)
    clocks = sampler.stop()

    def hbm_rate(batch, ctx, ms):
        return (weight_bytes_read_per_step(cfg) + batch * ctx * kv_bytes_per_token(cfg)) / (ms / 1e3) / 1e9

    achieved = hbm_rate(args.batch, mean_ctx, ms_step)
    flops = prefill_flops(cfg, PREFILL_LEN)
    kernels = {
        f"decode_b{args.batch}": kernel_rows(cfg, kinds8, peaks, args.batch, args.batch, mean_ctx, True),
        "decode_b64": {k: v for k, v in kernel_rows(cfg, kinds64, peaks, 64, 64, ctx64, True).items()
                       if k == "K5_decode_attention"},
        f"prefill_{PREFILL_LEN}": kernel_rows(cfg, kinds_prefill, peaks, PREFILL_LEN, 1, PREFILL_LEN, False),
        "how": "every kind of kernel by itself: a step's launches of that kind (one per layer, on that "
               "layer's weights and cache) back to back between two CUDA events, queued behind a busy "
               "device, L2 flushed before, median of 5, per launch; decode: bytes / time of the measured copy rate, prefill: flops / time of the "
               "measured burst bf16 rate",
    }
    return {
        "metric": METRIC,
        "value": round(tps, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights N(0, 0.02), uniform-random token ids",
        "impl": "ours",
        "config": {
            "model": "llama-3.2-1b-shape", "layers": cfg["num_hidden_layers"], "layers_run": layers_run,
            "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
            "global_batch": args.batch, "seq_len": PROMPT_LEN, "max_context": MAX_CONTEXT,
            "prefill_tokens": PREFILL_LEN, "block_size": BLOCK_SIZE, "parallelism": "single-gpu",
            "l2": "inputs larger than L2 (2.47 GB of weights per step)", "peaks": peaks_kind,
            "max_model_len": engine.max_model_len,
        },
        "e2e": {"value": round(e2e_tps, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "prefill": {"value": round(PREFILL_LEN / (prefill_ms / 1e3), 1), "tokens": PREFILL_LEN,
                    "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": {"decode_b1": round(b1, 1), "decode_b64": round(b64, 1),
                   "decode_b1_frac": round(hbm_rate(1, ctx1, ms1) / peaks["hbm_gbs"], 4),
                   "decode_b64_frac": round(hbm_rate(64, ctx64, ms64) / peaks["hbm_gbs"], 4)},
        "kernels": kernels,
        "gpu_launches": int(launches),
        "clocks": clocks,
    }


# --- the reference --------------------------------------------------------------------------------


class _StubTokenizer:
    """The reference's engine detokenises every token; with random weights there is no text,
    so decoding returns nothing (its own tests use a byte-level fake in the same place)."""

    def decode(self, ids, **_):
        return ""


def run_reference(args) -> dict:
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "engine").is_dir():
        return {"impl": "reference", "unavailable": "baseline/_ref holds no installed reference"}
    try:
        import torch

        sys.path.insert(0, str(ref))
        from engine.model.loader import load_model  # the reference's own loader
        from engine.runtime.engine import LLMEngine as RefEngine
        from engine.runtime.params import SamplingParams as RefParams

        from inference_engine_b200.weights import write_random_model

        torch.cuda.set_device(0)
        with tempfile.TemporaryDirectory(prefix="ie_b200_ref_") as tmp:
            write_random_model(dict(LLAMA_1B), tmp, seed=0)
            model = load_model(tmp, device="cuda", dtype=torch.bfloat16)
        blocks = -(-args.batch * (PROMPT_LEN + args.warmup + args.steps + 64) // BLOCK_SIZE)
        g = torch.Generator().manual_seed(2)
        prompts = torch.randint(0, LLAMA_1B["vocab_size"], (args.batch, PROMPT_LEN), generator=g).tolist()
        params = RefParams(temperature=0.0, max_tokens=args.warmup + args.steps + 8)

        def attempt(tag: str, batch: int, **mode):
            engine = RefEngine(model, _StubTokenizer(), (), num_blocks=blocks, block_size=BLOCK_SIZE,
                               max_num_seqs=max(batch, 8), max_num_batched_tokens=4 * PROMPT_LEN,
                               enable_prefix_caching=False, max_model_len=MAX_CONTEXT, **mode)
            for i, p in enumerate(prompts[:batch]):
                engine.add_request(f"ref-{tag}-{i}", p, params)
            produced = 0
            while produced < batch * args.warmup:
                produced += len(engine.step())
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            tokens = 0
            for _ in range(args.steps):
                tokens += len(engine.step())
            torch.cuda.synchronize()
            elapsed = time.perf_counter() - t0
            used_graph = bool(engine.step_log and engine.step_log[-1].get("graph"))
            for i in range(batch):
                engine.abort(f"ref-{tag}-{i}")
            return tokens, elapsed, used_graph

        def copies(batch: int, graph: bool) -> tuple[int, int]:
            """Bytes its step copies to the device and back, counted from the tensors it builds
            (a captured decode step: engine/runtime/cuda_graphs.py:87-108; an eager one:
            engine/runtime/paged_cache.py:98-123 and engine/runtime/engine.py:225-229); the
            tokens come back as one 64-bit integer per row (engine.py:229)."""
            ctx = PROMPT_LEN + args.warmup + args.steps // 2
            if graph:  # ids, positions, slots (64-bit), lengths and block tables (32-bit), padded to the bucket
                bucket = next(n for n in (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256) if n >= batch)
                return bucket * (3 * 8 + 4) + bucket * -(-ctx // BLOCK_SIZE) * 4, batch * 8
            # every cached position's slot per request, the new slots, starts, lengths (twice), ids, positions: 64-bit
            return 8 * (batch * ctx + batch + (batch + 1) + 2 * batch + 2 * batch), batch * 8

        sampler = ClockSampler()
        sampler.start()
        mode = "default (Triton decode kernel, CUDA graphs)"
        try:
            tokens, elapsed, used_graph = attempt("default", args.batch)
        except Exception as first:  # its fast path needs a newer torch than this image has
            mode = (f"eager (use_triton=False, its bench_decode.py 'eager' mode); the default mode "
                    f"raised {type(first).__name__}: {str(first)[:120]}")
            torch.cuda.synchronize()
            tokens, elapsed, used_graph = attempt("eager", args.batch, use_triton=False)
        # One request alone never meets the call that fails above (it is made for several prompts
        # in one step, and for its captured mixed steps), so batch 1 also runs with the reference's
        # fastest decode path: its Triton kernel inside captured decode steps.
        points = {}
        try:
            t1, e1, g1 = attempt("b1", 1, enable_mixed_graphs=False)
            points = {"decode_b1": round(t1 / e1, 1),
                      "decode_b1_mode": "Triton decode kernel%s, enable_mixed_graphs=False" % (", CUDA graphs" if g1 else "")}
        except Exception as exc:
            points = {"decode_b1": None, "decode_b1_mode": f"default mode raised {type(exc).__name__}: {str(exc)[:100]}"}
        clocks = sampler.stop()
        tps = tokens / elapsed
        h2d, d2h = copies(args.batch, used_graph)
        return {
            "metric": METRIC, "value": round(tps, 1),
            "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(elapsed / args.steps * 1e3, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "impl": "reference",
            "data": "synthetic: seeded random weights N(0, 0.02), uniform-random token ids",
            "config": {"model": "llama-3.2-1b-shape", "global_batch": args.batch,
                       "seq_len": PROMPT_LEN, "block_size": BLOCK_SIZE, "parallelism": "single-gpu",
                       "mode": mode,
                       "timing": "wall clock around LLMEngine.step(), synchronised on both sides"},
            "e2e": {"value": round(tps, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h},
            "points": points,
            "clocks": clocks,
        }
    except Exception as exc:  # the reference is other people's code on hardware it never saw
        return {"impl": "reference", "unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    result = run_reference(args) if args.impl == "reference" else run_ours(args)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
