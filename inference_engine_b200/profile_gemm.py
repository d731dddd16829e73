"""The bfloat16 products of a layer by themselves over row counts: what `CudaOps.linear` routes a
product to against the alternatives it has (the vendor library's plain product, the same cut along
the inner dimension into 2, 4 or 8 parts as one batched product, the few-row weight-streaming kernel).

    python -m inference_engine_b200.profile_gemm --rows 8,16,17,64,96,128,256,512
    python -m inference_engine_b200.profile_gemm --shapes qkv:3072x2048,down:2048x8192 --rows 64

A launch stands for one layer of a step: every launch takes the next of several weight matrices
(together larger than L2).  The launches of two rounds over the matrices are captured in one CUDA
graph and timed with CUDA events; the best of three replays counts.  One JSON line per (rows, shape):
microseconds per launch for every way, and how far the routed one is behind the best.
"""

from __future__ import annotations

import argparse
import json

SHAPES_1B = "qkv:3072x2048,out:2048x2048,gate_up:16384x2048,down:2048x8192"


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--rows", default="4,8,9,16,17,32,64,96,128,256,512")
    ap.add_argument("--shapes", default=SHAPES_1B, help="name:NxK, comma-separated (default: the 1B shape's four)")
    args = ap.parse_args()

    import torch

    from .engine.workspace import Workspace
    from .kernels import get_ops

    ops, ws = get_ops("cuda"), Workspace("cuda")

    def timed(fn, copies: int) -> float:
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        graph, iters = torch.cuda.CUDAGraph(), 2 * copies
        with torch.cuda.graph(graph):
            for i in range(iters):
                fn(i)
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
        return best

    shapes = []
    for item in args.shapes.split(","):
        name, dims = item.split(":")
        n, k = (int(v) for v in dims.lower().split("x"))
        shapes.append((name, n, k))
    for m in (int(v) for v in args.rows.split(",")):
        for name, n, k in shapes:
            copies = min(max(2, int(600e6 // (n * k * 2))), 24)
            weights = [(torch.randn(n, k, device="cuda") * 0.02).bfloat16() for _ in range(copies)]
            x = torch.randn(m, k, device="cuda").bfloat16()
            out = torch.empty(m, n, device="cuda", dtype=torch.float32)

            def routed(i):
                ops.linear(x, weights[i % copies], ws=ws, tag="t", out_dtype=torch.float32, allow_split=True)

            us = {"routed": timed(routed, copies),
                  "library": timed(lambda i: torch.mm(x, weights[i % copies].t(), out_dtype=torch.float32, out=out), copies)}
            for parts in (2, 4, 8):
                if k % (parts * 64) == 0 and k // parts >= 256:
                    ks = k // parts
                    cut = torch.empty(parts, m, n, device="cuda", dtype=torch.float32)
                    us[f"library_{parts}_parts"] = timed(
                        lambda i: torch.bmm(x.view(m, parts, ks).permute(1, 0, 2),
                                            weights[i % copies].view(n, parts, ks).permute(1, 2, 0),
                                            out_dtype=torch.float32, out=cut), copies)
            if m <= ops.FEW_ROWS:
                saved, ops.blas_split_k = ops.blas_split_k, False
                try:
                    us["few_row_kernel"] = timed(routed, copies)
                finally:
                    ops.blas_split_k = saved
            best = min(us, key=us.get)
            print(json.dumps({"rows": m, "product": name, "n": n, "k": k,
                              "us": {key: round(v, 2) for key, v in us.items()}, "best": best,
                              "routed_behind": round(us["routed"] / us[best] - 1, 3)}), flush=True)
            del weights
    ops.check_errors()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
