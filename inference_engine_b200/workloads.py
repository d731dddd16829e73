"""Continuous-batching workloads on random-weight Llama shapes, through ``LLMEngine`` as a user
drives it (requests in, ``step()`` until done).  Three of them:

    python -m inference_engine_b200.workloads 1b   # 32 requests, prompts of 128..4096 tokens, 256 new tokens each
    python -m inference_engine_b200.workloads 3b   # the same requests on the 3B shape, portions of 512 tokens
    python -m inference_engine_b200.workloads 8b   # 64 requests of 2048 tokens, 512 new tokens each, on the 8B
                                                   # shape, with a cache too small for all of them (preemption)
    python -m inference_engine_b200.workloads chat # 1B shape: 192 requests with prompts of 16..200 tokens and 64 new
                                                   # tokens each; a new one arrives every second step, so every
                                                   # other step holds a prompt beside up to 32 decoding requests

``--chunk`` sets the token budget of a step (the size of prompt portions); ``--no-mixed-graphs`` launches
steps that hold prompt portions eagerly (decode steps stay captured).  Every workload runs three
times; the last run (warm: kernels built, launch sequences captured) is the one to read.  One JSON line
per run.
"""

from __future__ import annotations

import argparse
import json
import time


def _shape(layers, hidden, heads, kv_heads, head_dim, intermediate, rope_factor, tied):
    return {
        "architectures": ["LlamaForCausalLM"], "num_hidden_layers": layers, "hidden_size": hidden,
        "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": head_dim,
        "intermediate_size": intermediate, "vocab_size": 128256, "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": rope_factor, "low_freq_factor": 1.0,
                         "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
        "rms_norm_eps": 1e-5, "tie_word_embeddings": tied, "max_position_embeddings": 131072,
    }


SHAPES = {
    "1b": _shape(16, 2048, 32, 8, 64, 8192, 32.0, True),
    "3b": _shape(28, 3072, 24, 8, 128, 8192, 32.0, True),
    "8b": _shape(32, 4096, 32, 8, 128, 14336, 8.0, False),
}


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("workload", choices=sorted(SHAPES) + ["chat"])
    ap.add_argument("--no-mixed-graphs", action="store_true")
    ap.add_argument("--chunk", type=int, default=None, help="token budget of a step (default: 4096; 3b: 512)")
    ap.add_argument("--runs", type=int, default=3)
    args = ap.parse_args()

    import torch

    from .engine.llm_engine import LLMEngine
    from .sampling.params import SamplingParams

    g = torch.Generator().manual_seed(0)
    block = 16
    shape = SHAPES["1b" if args.workload == "chat" else args.workload]
    arrive_every = 0  # steps between two arrivals (0: all requests are there from the start)
    if args.workload == "chat":
        lengths = torch.randint(16, 201, (192,), generator=g).tolist()
        new_tokens, seqs, arrive_every = 64, 32, 2
        num_blocks = seqs * (200 + new_tokens + 2 * block) // block + 64
        chunk = args.chunk or 4096
    elif args.workload == "8b":
        lengths, new_tokens, seqs = [2048] * 64, 512, 64
        # room for 70 % of what all requests hold at their longest: some are preempted and prefilled again
        num_blocks = int(seqs * (2048 + new_tokens) * 0.7) // block
        chunk = args.chunk or 4096
    else:
        lengths = torch.randint(128, 4097, (32,), generator=g).tolist()
        new_tokens, seqs = 256, 32
        num_blocks = (sum(lengths) + seqs * (new_tokens + 2 * block)) // block + 64
        chunk = args.chunk or (512 if args.workload == "3b" else 4096)
    vocab = shape["vocab_size"]
    prompts = {f"r{i}": torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(lengths)}
    engine = LLMEngine.from_random(shape, seed=0, dtype="bfloat16", device="cuda", max_model_len=8192,
                                   block_size=block, num_blocks=num_blocks, max_num_seqs=seqs,
                                   max_num_batched_tokens=chunk, enable_cuda_graphs=True,
                                   enable_mixed_graphs=not args.no_mixed_graphs)
    params = SamplingParams(temperature=0, max_tokens=new_tokens)
    for run in range(args.runs):
        waiting = [(f"{rid}-{run}", prompt) for rid, prompt in prompts.items()]
        if not arrive_every:
            for rid, prompt in waiting:
                engine.add_request(rid, prompt, params)
            waiting = []
        preempted = engine.scheduler.num_preemptions
        steps = produced = 0
        seconds = {"decode": 0.0, "with_prompt_portions": 0.0}
        counts = {"decode": 0, "with_prompt_portions": 0}
        torch.cuda.synchronize()
        started = time.perf_counter()
        while waiting or engine.has_unfinished():
            if waiting and (steps % arrive_every == 0 or not engine.has_unfinished()):
                engine.add_request(*waiting.pop(0), params)
            t0 = time.perf_counter()
            produced += len(engine.step())
            kind = "with_prompt_portions" if engine.step_log[-1]["prefill_tokens"] > 0 else "decode"
            seconds[kind] += time.perf_counter() - t0
            counts[kind] += 1
            steps += 1
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - started
        engine.ops.check_errors()
        print(json.dumps({
            "workload": args.workload, "run": run, "requests": len(prompts), "prompt_tokens": sum(lengths),
            "new_tokens": produced, "chunk": chunk, "seconds": round(elapsed, 3), "steps": steps,
            "new_tokens_per_s": round(produced / elapsed, 1),
            "all_tokens_per_s": round((produced + sum(lengths)) / elapsed, 1),
            "preemptions": engine.scheduler.num_preemptions - preempted,
            "mixed_graphs": engine.mixed_graphs is not None,
            "steps_by_kind": counts, "seconds_by_kind": {k: round(v, 3) for k, v in seconds.items()},
        }), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
