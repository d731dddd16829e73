"""The decode attention kernel by itself over batches and context lengths: microseconds per launch and
the fraction of a memory bandwidth at which it reads the keys and values it must read.

    python -m inference_engine_b200.profile_attention --cases 8x1024,64x1024,64x4096,16x16384,1x32768
    IE_B200_DECODE_NARROW=0 python -m inference_engine_b200.profile_attention   # the 16-row layout for all

Every request brings one token.  A launch stands for one layer of a step: it runs on a cache of its own
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
    args = ap.parse_args()

    import torch

    from .engine.workspace import Workspace
    from .kernels import get_ops

    ops = get_ops("cuda")
    nh, nkv, hd, ps = args.heads, args.kv_heads, args.head_dim, args.page_size
    peak = args.peak_gbs or _peak_gbs()

    def case(batch: int, ctx_len: int, ws):
        pages_per = -(-ctx_len // ps)
        total = batch * pages_per + 2
        perm = torch.randperm(total, device="cuda").to(torch.int32)
        tables = perm[: batch * pages_per].view(batch, pages_per).contiguous()
        k = torch.randn(total, nkv, ps, hd, device="cuda").bfloat16()
        v = torch.randn_like(k)
        q = torch.randn(batch, nh * hd, device="cuda").bfloat16()
        ctx = types.SimpleNamespace(
            num_tokens=batch, num_seqs=batch, q_lens=[1] * batch, max_q_len=1, max_ctx_len=ctx_len, ws=ws,
            positions=torch.full((batch,), ctx_len - 1, dtype=torch.int32, device="cuda"),
            seq_of_token=torch.arange(batch, dtype=torch.int32, device="cuda"),
            cu_q=torch.arange(batch + 1, dtype=torch.int32, device="cuda"),
            ctx_lens=torch.full((batch,), ctx_len, dtype=torch.int32, device="cuda"))
        return q, k, v, tables, ctx

    for item in args.cases.split(","):
        batch, ctx_len = (int(x) for x in item.lower().split("x"))
        ws = Workspace("cuda")
        visible = min(ctx_len, args.window) if args.window > 0 else ctx_len  # keys a request's token sees
        kv_bytes = batch * visible * nkv * hd * 2 * 2
        cases = [case(batch, ctx_len, ws) for _ in range(max(2, min(8, int(1.0e9 // (batch * ctx_len * nkv * hd * 4)))))]
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
        row = {"requests": batch, "context": ctx_len, "us": round(best, 2), "gbs": round(gbs, 1),
               "caches": len(cases), "kv_mb_per_launch": round(kv_bytes / 1e6, 1)}
        if peak:
            row["frac"] = round(gbs / peak, 3)
        print(json.dumps(row), flush=True)
        del cases, graph
        torch.cuda.empty_cache()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
