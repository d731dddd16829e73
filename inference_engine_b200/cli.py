"""Command line: ``engine info``, ``engine generate``, ``engine replay``.

Option names and meanings are the reference's (engine/cli.py:142-197) where it has them:
``--model``, ``--prompt``, ``--temperature`` (0.7), ``--top-p`` (0.9), ``--max-tokens`` (256),
``--seed``, ``--device``, ``--gpu-mem`` and, from its ``serve`` command, ``--dtype``,
``--max-num-seqs``, ``--max-num-batched-tokens``, ``--block-size``, ``--num-blocks``,
``--gpu-memory-utilization``, ``--no-chunked-prefill``, ``--no-cuda-graphs``, ``--no-mixed-graphs``.  There is no
``serve``.  ``generate`` takes token ids (``--prompt-ids``) when the model folder has no
tokenizer, and can run a named-size random model (``--random-config FILE``).
"""

from __future__ import annotations

import argparse
import json
import sys
import time

GIB = 2**30


def cmd_info(args: argparse.Namespace) -> int:
    """Model shape and whether it fits a GPU of --gpu-mem GiB.  What is printed comes from the
    architecture's registry entry; an architecture that registered no footprint is built
    (without weights) and counted."""
    from .config import build_model_spec, get_architecture, load_config

    cfg = load_config(args.model)
    arch = get_architecture(cfg.architecture)
    for line in (arch.describe(cfg) if arch.describe else [f"architecture        {cfg.architecture}"]):
        print(line)
    if arch.footprint is not None:
        footprint = arch.footprint(cfg)
    else:
        from .engine.model import Model

        footprint = Model(build_model_spec(cfg), "bfloat16", max_positions=1).footprint()
        print(f"parameters          {footprint.parameters / 1e9:.3f} B")
        print(f"cache per token     {footprint.cache_bytes_per_token(2) / 1024:.1f} KiB (bf16)")
    if footprint.state_values_per_request:
        print(f"state per request   {footprint.state_values_per_request * 4 / 1024:.1f} KiB (fp32)")
    print(f"\nOn a {args.gpu_mem:g} GiB GPU (1 GiB reserved for activations and CUDA context):")
    for label, bytes_per_param in (("bf16", 2.0), ("fp32", 4.0)):
        tokens = footprint.cache_tokens_that_fit(args.gpu_mem, bytes_per_param,
                                                 cache_dtype_bytes=int(bytes_per_param))
        verdict = f"{tokens:>11,} KV tokens fit" if tokens else "        does not fit"
        print(f"  {label}  weights {footprint.parameters * bytes_per_param / GIB:6.1f} GiB  ->{verdict}")
    return 0


def _engine_config(args: argparse.Namespace):
    from .config import EngineConfig

    return EngineConfig(
        dtype=args.dtype, num_blocks=args.num_blocks, block_size=args.block_size, max_num_seqs=args.max_num_seqs,
        max_num_batched_tokens=args.max_num_batched_tokens,
        gpu_memory_utilization=args.gpu_memory_utilization,
        enable_chunked_prefill=not args.no_chunked_prefill,
        enable_cuda_graphs=False if args.no_cuda_graphs else None,
        enable_mixed_graphs=False if args.no_cuda_graphs or args.no_mixed_graphs else None,
        max_model_len=args.max_model_len,
    )


def cmd_generate(args: argparse.Namespace) -> int:
    from .engine.llm_engine import LLMEngine
    from .sampling.params import SamplingParams

    tokenizer = None
    if args.random_config:
        with open(args.random_config, encoding="utf-8") as f:
            engine = LLMEngine.from_random(json.load(f), args.seed or 0, device=args.device,
                                           config=_engine_config(args))
    else:
        if args.model is None:
            raise SystemExit("engine generate: --model or --random-config is required")
        if args.prompt is not None:
            from transformers import AutoTokenizer  # tokenizer only; the model code is ours

            tokenizer = AutoTokenizer.from_pretrained(args.model)
        engine = LLMEngine.from_model_dir(args.model, device=args.device, tokenizer=tokenizer,
                                          config=_engine_config(args))
    print(f"[engine] {engine.dtype}, max_model_len {engine.max_model_len}, "
          f"{engine.cache.pools[0].num_pages if engine.cache.pools else 0} cache pages of "
          f"{engine.cache.page_size} tokens, captured decode steps {'on' if engine.graphs else 'off'}",
          file=sys.stderr)
    if args.prompt is not None and tokenizer is not None:
        messages = [{"role": "user", "content": args.prompt}]
        if getattr(tokenizer, "chat_template", None):
            prompt_ids = list(tokenizer.apply_chat_template(messages, add_generation_prompt=True))
        else:
            prompt_ids = list(tokenizer.encode(args.prompt))
    elif args.prompt_ids:
        prompt_ids = [int(t) for t in args.prompt_ids.replace(",", " ").split()]
    elif args.prompt_len:
        import random

        rng = random.Random(args.seed or 0)
        prompt_ids = [rng.randrange(engine.model.spec.vocab_size) for _ in range(args.prompt_len)]
    else:
        raise SystemExit("engine generate: give --prompt (needs a tokenizer in the model folder), "
                         "--prompt-ids or --prompt-len")
    params = SamplingParams(temperature=args.temperature, top_p=args.top_p,
                            max_tokens=args.max_tokens, seed=args.seed)
    engine.add_request("cli", prompt_ids, params)
    start, n_tokens, ids = time.perf_counter(), 0, []
    while engine.has_unfinished():
        for out in engine.step():
            n_tokens += 1
            ids.append(out.token_id)
            if tokenizer is not None:
                print(out.text, end="", flush=True)
    if tokenizer is None:
        print(" ".join(map(str, ids)))
    elapsed = time.perf_counter() - start
    print(f"\n\n[{n_tokens} tokens in {elapsed:.2f}s, {n_tokens / elapsed:.1f} tokens/s]",
          file=sys.stderr)
    return 0


def cmd_replay(args: argparse.Namespace) -> int:
    """The trace replay program (what ``bin/trace_run`` runs)."""
    from .engine.replay import main as replay_main

    return replay_main(["--model", args.model, "--dtype", args.dtype, "--out", args.out,
                        "--max-tokens", str(args.max_tokens), "--block-size", str(args.block_size)])


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="engine", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = parser.add_subparsers(dest="command", required=True)

    info = sub.add_parser("info", help="show model shape and GPU memory fit")
    info.add_argument("--model", required=True, help="local model directory")
    info.add_argument("--gpu-mem", type=float, default=180.0, help="GPU memory in GiB")
    info.set_defaults(func=cmd_info)

    gen = sub.add_parser("generate", help="completion for one prompt, streamed")
    gen.add_argument("--model", default=None)
    gen.add_argument("--random-config", default=None,
                     help="a config.json file: run that shape with seeded random weights")
    gen.add_argument("--prompt", default=None, help="text (needs a tokenizer in the model folder)")
    gen.add_argument("--prompt-ids", default=None, help="token ids, comma or space separated")
    gen.add_argument("--prompt-len", type=int, default=None, help="that many seeded random ids")
    gen.add_argument("--temperature", type=float, default=0.7)
    gen.add_argument("--top-p", type=float, default=0.9)
    gen.add_argument("--max-tokens", type=int, default=256)
    gen.add_argument("--seed", type=int, default=None)
    gen.add_argument("--device", default="cuda")
    gen.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    gen.add_argument("--max-num-seqs", type=int, default=64, help="max running sequences")
    gen.add_argument("--max-num-batched-tokens", type=int, default=4096)
    gen.add_argument("--block-size", type=int, default=16)
    gen.add_argument("--num-blocks", type=int, default=None, help="default: fill free GPU memory")
    gen.add_argument("--gpu-memory-utilization", type=float, default=0.9)
    gen.add_argument("--max-model-len", type=int, default=None)
    gen.add_argument("--no-chunked-prefill", action="store_true")
    gen.add_argument("--no-cuda-graphs", action="store_true")
    gen.add_argument("--no-mixed-graphs", action="store_true",
                     help="short steps with prompt portions run eagerly (decode steps stay captured)")
    gen.set_defaults(func=cmd_generate)

    rep = sub.add_parser("replay", help="feed token ids step by step (stdin) and write logits")
    rep.add_argument("--model", required=True)
    rep.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    rep.add_argument("--out", required=True)
    rep.add_argument("--max-tokens", type=int, required=True)
    rep.add_argument("--block-size", type=int, default=16)
    rep.set_defaults(func=cmd_replay)
    return parser


def main(argv: list[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    return args.func(args)


if __name__ == "__main__":
    raise SystemExit(main())
