"""A steady-state driver for profilers: a few decode steps, one prefill, or a step with a prompt's last
portion beside decoding requests (``--mode mixed``), of a random-weight Llama shape, launched eagerly (no captured launch sequence) so that every kernel shows up by
name.  The reference has bench/profile_step.py in this role.

    python -m inference_engine_b200.profile_step --mode decode --batch 8 --context 1024 --layers 4
    ncu --metrics gpu__time_duration.sum --clock-control none --csv --log-file launches.csv \\
        python -m inference_engine_b200.profile_step --mode decode --batch 8 --layers 2 --steps 2

With ``--events`` it prints the device time per step measured with CUDA events instead.
``--phase-clocks`` (prefill, head sizes 64 and 128) builds the tcgen05 prefill attention with clock stamps
around the phases of one softmax thread (``-DIE_TC5_TIMING``) and prints the clocks per key tile that thread
spent in each: where a query row's time goes between two key tiles.
"""

from __future__ import annotations

import argparse
import json


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--mode", choices=["decode", "prefill", "mixed"], default="decode",
                    help="mixed: the last --tokens tokens of a --prompt-token prompt beside batch - 1 decoding requests")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=1024, help="tokens cached per request (decode)")
    ap.add_argument("--tokens", type=int, default=2048, help="prompt tokens (prefill), tokens of the portion (mixed)")
    ap.add_argument("--prompt-tokens", type=int, default=4096, help="length of the prompt whose last portion runs (mixed)")
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--config", default=None, help="a config.json file (default: Llama 3.2 1B shape)")
    ap.add_argument("--graphs", action="store_true", help="replay captured decode steps")
    ap.add_argument("--phase-clocks", action="store_true",
                    help="prefill: clocks per key tile in each phase of a softmax thread of the tcgen05 attention")
    args = ap.parse_args()
    if args.phase_clocks:  # (before the kernels are built: the flag is part of the library's name)
        import os

        os.environ["IE_B200_NVCC_FLAGS"] = (os.environ.get("IE_B200_NVCC_FLAGS", "") + " -DIE_TC5_TIMING").strip()

    import torch

    from .engine.batch import StepEntry
    from .engine.llm_engine import LLMEngine

    if args.config:
        with open(args.config, encoding="utf-8") as f:
            cfg = json.load(f)
    else:
        cfg = {
            "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 16, "hidden_size": 2048,
            "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
            "intermediate_size": 8192, "vocab_size": 128256, "rope_theta": 500000.0,
            "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                             "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
            "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 131072,
        }
    cfg["num_hidden_layers"] = args.layers
    block = 16
    per_req = {"decode": args.context, "prefill": args.tokens,
               "mixed": max(args.context, args.prompt_tokens)}[args.mode] + args.steps + args.warmup + 16
    engine = LLMEngine.from_random(
        cfg, seed=0, dtype=args.dtype, device="cuda", max_model_len=max(per_req, 64),
        num_blocks=args.batch * (-(-per_req // block) + 1), block_size=block,
        max_num_seqs=args.batch, max_num_batched_tokens=max(args.tokens, args.batch, 2048),
        enable_cuda_graphs=args.graphs)
    runner, cache, vocab = engine.runner, engine.cache, cfg["vocab_size"]
    g = torch.Generator().manual_seed(0)
    times = []
    if args.mode == "prefill":
        for r in range(args.warmup + args.steps):
            prompt = torch.randint(0, vocab, (args.tokens,), generator=g).tolist()
            cache.add_request(r)
            cache.grow(r, 0, args.tokens)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            runner.step([StepEntry(r, prompt, 0, [args.tokens - 1])])
            e.record()
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e))
            cache.free(r)
    elif args.mode == "mixed":
        chunk = 2048
        cache.add_request("prompt")
        cache.grow("prompt", 0, args.prompt_tokens)
        done = args.prompt_tokens - args.tokens
        for start in range(0, done, chunk):
            n = min(chunk, done - start)
            runner.step([StepEntry("prompt", torch.randint(0, vocab, (n,), generator=g).tolist(), start, [])])
        ids = list(range(args.batch - 1))
        for rid in ids:
            cache.add_request(rid)
            cache.grow(rid, 0, args.context + 1)
            for start in range(0, args.context, chunk):
                n = min(chunk, args.context - start)
                runner.step([StepEntry(rid, torch.randint(0, vocab, (n,), generator=g).tolist(), start, [])])
        portion = torch.randint(0, vocab, (args.tokens,), generator=g).tolist()
        entries = [StepEntry("prompt", portion, done, [args.tokens - 1])]
        entries += [StepEntry(rid, [int(torch.randint(0, vocab, (1,), generator=g))], args.context, [0]) for rid in ids]
        for k in range(args.warmup + args.steps):  # the same step again and again: it writes the same cache slots
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            runner.step(entries)
            e.record()
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e))
    else:
        ids = list(range(args.batch))
        for rid in ids:
            cache.add_request(rid)
            cache.grow(rid, 0, args.context)
        chunk = 2048
        for rid in ids:  # fill the cache with real keys and values
            for start in range(0, args.context, chunk):
                n = min(chunk, args.context - start)
                runner.step([StepEntry(rid, torch.randint(0, vocab, (n,), generator=g).tolist(), start, [])])
        out = torch.empty(args.batch, dtype=torch.int32, device="cuda")
        pos = args.context
        for k in range(args.warmup + args.steps):
            for rid in ids:
                cache.grow(rid, pos, pos + 1)
            entries = [StepEntry(rid, [int(torch.randint(0, vocab, (1,), generator=g))], pos, [0]) for rid in ids]
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            logits = engine.graphs.run(entries) if engine.graphs is not None else runner.step(entries)
            engine.ops.argmax(logits, out)
            e.record()
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e))
            pos += 1
    engine.ops.check_errors()
    if args.phase_clocks and args.mode == "prefill":
        import ctypes

        lib = engine.ops._attention_lib(cfg["head_dim"])
        clocks = (ctypes.c_longlong * 16)()
        lib.ie_tc5_timing(clocks, 1)  # forget the warm-up
        rid = "phase-clocks"
        cache.add_request(rid)
        cache.grow(rid, 0, args.tokens)
        runner.step([StepEntry(rid, torch.randint(0, vocab, (args.tokens,), generator=g).tolist(), 0, [])])
        torch.cuda.synchronize()
        lib.ie_tc5_timing(clocks, 1)
        tiles = max(clocks[15], 1)
        names = ["loop top (with the stamps' own cost)", "wait for S = Q K^T", "read the row of S (tcgen05.ld)",
                 "mask, maximum, vote", "exponentials, sum, pack", "write the weights (tcgen05.st)",
                 "wait for the previous P V (and rescale)", "fence and arrive"]
        print(json.dumps({"phase_clocks_per_key_tile": {n: round(clocks[i] / tiles) for i, n in enumerate(names)},
                          "key_tiles_of_the_stamped_block": int(clocks[15]), "layers": args.layers}))
    steady = times[args.warmup:]
    print(json.dumps({"mode": args.mode, "batch": args.batch, "layers": args.layers,
                      "ms_per_step": [round(t, 4) for t in steady]}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
