"""The decode attention kernel by itself over batches and context lengths: microseconds per launch and
the fraction of a memory bandwidth at which it reads the keys and values it must read.

    python -m inference_engine_b200.profile_attention --cases 8x1024,64x1024,64x4096,16x16384,1x32768
    IE_B200_DECODE_NARROW=0 python -m inference_engine_b200.profile_attention   # the 16-row layout for all
    python -m inference_engine_b200.profile_attention --cases 32x128-4352       # 32 contexts of 128 to 4,352 tokens
    python -m inference_engine_b200.profile_attention --cases 8000+7*500        # one of 8,000 tokens and seven of 500
    IE_B200_DECODE_BALANCED=0 python -m inference_engine_b200.profile_attention --cases 32x128-4352   # dealt by request

Every request brings one token (``--portion T``: its last T tokens, a prompt portion for the prefill kernel; the row
then gives TFLOP/s).  ``BxL`` is B requests of L cached tokens, ``BxL1-L2`` B requests whose lengths
are drawn evenly from L1 to L2 (seeded); which of the two decode kernels runs is the engine's own choice
(``CudaOps.decode_dealing``) unless ``IE_B200_DECODE_BALANCED`` (by length: 0, 1) or ``IE_B200_DECODE_SMALL`` (no blocks of 2 or 3 warps: 0) says otherwise.  A launch stands for one layer of a step: it runs on a cache of its own
(several caches, together larger than L2, taken in turn), block tables point at shuffled pages.  The launches
of four rounds over the caches are captured in one CUDA graph and timed with CUDA events; the best of
three replays counts.  ``--peak-gbs`` is the bandwidth the fraction is of (default: the copy rate in
MEASURED_PEAKS.json beside the package, if there is one).
"""

from __future__ import annotations

import argparse
import json
import types
from pathlib import Path


def _peak_gbs() -> float | None:
    path = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(path.read_text())["hbm_gbs"])
    except (OSError, ValueError, KeyError):
        return None


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--cases", default="8x1024,64x1024,32x2304,64x4096,16x16384,1x32768",
                    help="requests x context length, comma-separated")
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--window", type=int, default=0)
    ap.add_argument("--peak-gbs", type=float, default=None)
    ap.add_argument("--caches", type=int, default=0, help="caches taken in turn (default: 2 to 8, about 1 GB in all)")
    ap.add_argument("--portion", type=int, default=1,
                    help="tokens every request brings, the last of its context (more than 16 / heads per group: the prefill kernel)")
    args = ap.parse_args()

    import torch

    from .engine.workspace import Workspace
    from .kernels import get_ops

    ops = get_ops("cuda")
    nh, nkv, hd, ps = args.heads, args.kv_heads, args.head_dim, args.page_size
    peak = args.peak_gbs or _peak_gbs()

    def case(lengths: list[int], ws):
        batch = len(lengths)
        pages = [-(-n // ps) for n in lengths]
        total, width = sum(pages) + 2, max(pages)
        perm = torch.randperm(total, device="cuda").to(torch.int32)
        tables = torch.full((batch, width), -1, dtype=torch.int32, device="cuda")
        at = 0
        for i, n in enumerate(pages):
            tables[i, :n] = perm[at: at + n]
            at += n
        k = torch.randn(total, nkv, ps, hd, device="cuda").bfloat16()
        v = torch.randn_like(k)
        t = args.portion
        q = torch.randn(batch * t, nh * hd, device="cuda").bfloat16()
        ragged = int(ops.decode_dealing(lengths, nkv, hd)) if batch > 1 and t == 1 else 0
        ctx = types.SimpleNamespace(
            num_tokens=batch * t, num_seqs=batch, q_lens=[t] * batch, max_q_len=t, max_ctx_len=max(lengths), ws=ws,
            positions=torch.tensor([n - t + i for n in lengths for i in range(t)], dtype=torch.int32, device="cuda"),
            seq_of_token=torch.arange(batch, dtype=torch.int32, device="cuda").repeat_interleave(t),
            cu_q=torch.arange(batch + 1, dtype=torch.int32, device="cuda") * t,
            ctx_lens=torch.tensor(lengths, dtype=torch.int32, device="cuda"), ragged=(ragged,),
            # (as the engine packs a step: the by-request kernel starts the longest requests' blocks first)
            decode_order=torch.tensor(sorted(range(batch), key=lambda i: -lengths[i]), dtype=torch.int32, device="cuda"))
        return q, k, v, tables, ctx

    for item in args.cases.split(","):
        if "+" in item:  # the lengths themselves, and "7*500" for seven of one length
            lengths = []
            for part in item.split("+"):
                times, _, n = part.rpartition("*")
                lengths += [int(n)] * (int(times) if times else 1)
            batch, length = len(lengths), item
        else:
            count, length = item.lower().split("x")
            batch = int(count)
        if "+" in item:
            pass
        elif "-" in length:
            low, high = (int(x) for x in length.split("-"))
            lengths = torch.randint(low, high + 1, (batch,), generator=torch.Generator().manual_seed(0)).tolist()
        else:
            lengths = [int(length)] * batch
        ctx_len = max(lengths)
        ws = Workspace("cuda")
        visible = [min(n, args.window) if args.window > 0 else n for n in lengths]  # keys a request's token sees
        kv_bytes = sum(visible) * nkv * hd * 2 * 2
        copies = args.caches or max(2, min(8, int(1.0e9 // (sum(lengths) * nkv * hd * 4))))
        cases = [case(lengths, ws) for _ in range(copies)]
        out = torch.empty_like(cases[0][0])

        def run(i: int) -> None:
            q, k, v, tables, ctx = cases[i % len(cases)]
            ops.paged_attention(q, k, v, tables, ctx, nh, nkv, hd, ps, hd ** -0.5, args.window, out)

        for i in range(3):
            run(i)
        torch.cuda.synchronize()
        ops.check_errors()
        graph, iters = torch.cuda.CUDAGraph(), len(cases) * 4
        with torch.cuda.graph(graph):
            for i in range(iters):
                run(i)
        graph.replay()
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(3):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            graph.replay()
            end.record()
            torch.cuda.synchronize()
            best = min(best, start.elapsed_time(end) / iters * 1e3)
        gbs = kv_bytes / best / 1e3
        row = {"requests": batch, "context": length, "dealt": ("by request", "by length", "by request, 2-warp blocks", "by request, 3-warp blocks")[cases[0][4].ragged[0]], "us": round(best, 2), "gbs": round(gbs, 1),
               "caches": len(cases), "kv_mb_per_launch": round(kv_bytes / 1e6, 1)}
        if args.portion > 1:  # (a portion's cost is its products: two per query and visible key, 2 hd flops each)
            seen = sum(min(n - args.portion + i + 1, args.window or n) for n in lengths for i in range(args.portion))
            row = {"requests": batch, "context": length, "portion": args.portion, "us": round(best, 2),
                   "tflops": round(4 * hd * nh * seen / best / 1e6, 1), "caches": len(cases)}
        elif peak:
            row["frac"] = round(gbs / peak, 3)
        print(json.dumps(row), flush=True)
        del cases, graph
        torch.cuda.empty_cache()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
