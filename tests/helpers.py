"""Shared test utilities: tiny random Llama weights, model folders, traces and comparison."""

from __future__ import annotations

import json
import random
from pathlib import Path

import torch

from tests import plain_llama


def llama_tensor_shapes(cfg: dict) -> dict[str, tuple[int, ...]]:
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads") or nh
    hd = cfg.get("head_dim") or h // nh
    shapes = {"model.embed_tokens.weight": (v, h), "model.norm.weight": (h,)}
    if not cfg.get("tie_word_embeddings", False):
        shapes["lm_head.weight"] = (v, h)
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}"
        shapes[f"{p}.self_attn.q_proj.weight"] = (nh * hd, h)
        shapes[f"{p}.self_attn.k_proj.weight"] = (nkv * hd, h)
        shapes[f"{p}.self_attn.v_proj.weight"] = (nkv * hd, h)
        shapes[f"{p}.self_attn.o_proj.weight"] = (h, nh * hd)
        shapes[f"{p}.mlp.gate_proj.weight"] = (i, h)
        shapes[f"{p}.mlp.up_proj.weight"] = (i, h)
        shapes[f"{p}.mlp.down_proj.weight"] = (h, i)
        shapes[f"{p}.input_layernorm.weight"] = (h,)
        shapes[f"{p}.post_attention_layernorm.weight"] = (h,)
    return shapes


def make_weights(cfg: dict, seed: int = 0, sharp: float = 3.0, std: float = 0.05) -> dict:
    """Random weights, stored as bfloat16 values.  Matrices are N(0, std), norm weights
    1 + N(0, std).  Query and key projections are scaled by ``sharp`` so that attention is
    peaked: with flat attention a lost or misplaced key changes the output by one part in
    hundreds and a cache fault would hide in the tolerance."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in llama_tensor_shapes(cfg).items():
        t = torch.randn(shape, generator=g) * std
        if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
            t = t + 1.0
        if name.endswith("q_proj.weight") or name.endswith("k_proj.weight"):
            t = t * sharp
        out[name] = t.to(torch.bfloat16)
    return out


def write_model_dir(path: Path, cfg: dict, weights: dict) -> Path:
    from safetensors.torch import save_file

    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(path / "model.safetensors"))
    return path


def random_tokens(cfg: dict, n: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist()


# --- traces --------------------------------------------------------------------------------------


def round64(n: int) -> int:
    return -(-n // 64) * 64


def trace_whole(requests: dict[str, list[int]]) -> list[dict]:
    return [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
             "end": [rid]} for i, (rid, toks) in enumerate(requests.items())]


def trace_decode_tail(requests: dict[str, list[int]], tail: int = 32) -> list[dict]:
    steps = []
    for rid, toks in requests.items():
        head = max(len(toks) - tail, 1)
        steps.append({"step": len(steps), "entries": [
            {"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        for p in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [
                {"id": rid, "tokens": [toks[p]], "want": [0]}], "end": []})
        steps[-1]["end"] = [rid]
    return steps


def trace_portions(requests: dict[str, list[int]], sizes=(7, 2, 19, 3, 2, 33, 5, 2, 16, 17)) -> list[dict]:
    steps = []
    for rid, toks in requests.items():
        pos, k = 0, 0
        while pos < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - pos)
            if len(toks) - pos - n == 1:  # never leave a single token: portions go down to two
                n += 1
            steps.append({"step": len(steps), "entries": [
                {"id": rid, "tokens": toks[pos:pos + n], "want": list(range(n))}], "end": []})
            pos, k = pos + n, k + 1
        steps[-1]["end"] = [rid]
    return steps


def trace_mixed(requests: dict[str, list[int]], seed: int = 0, live_max: int = 4,
                tail: int = 12, max_portion: int = 24) -> tuple[list[dict], int]:
    """Up to ``live_max`` requests alive at once: portions of some beside single decoded
    tokens of others, requests sometimes left out of a step, new ones admitted as old ones
    end.  Returns the steps and the largest number of tokens (each request rounded up to a
    multiple of 64) that live requests hold at any time."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live: dict[str, int] = {}
    steps, peak = [], 0
    while waiting or live:
        while waiting and len(live) < live_max and (not live or rng.random() < 0.6):
            rid, _ = waiting.pop(0)
            live[rid] = 0
        peak = max(peak, sum(round64(len(requests[r])) for r in live))
        entries, ended = [], []
        for rid in list(live):
            toks, pos = requests[rid], live[rid]
            if len(live) > 1 and rng.random() < 0.2:
                continue  # left out of this step
            remaining = len(toks) - pos
            if remaining <= tail:
                n = 1
            else:
                n = min(rng.randint(2, max_portion), remaining - tail)
                if n == 1:
                    n = 2 if remaining - tail >= 2 else 1
            entries.append({"id": rid, "tokens": toks[pos:pos + n], "want": list(range(n))})
            live[rid] = pos + n
            if live[rid] == len(toks):
                ended.append(rid)
                del live[rid]
        if entries:
            rng.shuffle(entries)
            steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps, peak


def restrict_wants(steps: list[dict], wanted: dict[str, set[int]]) -> list[dict]:
    """The same steps, asking only for the logits at the positions in ``wanted`` (per request:
    positions within the whole request).  For large vocabularies, where every position's logits
    would be gigabytes."""
    fed: dict[str, int] = {}
    out = []
    for step in steps:
        entries = []
        for e in step["entries"]:
            start = fed.get(e["id"], 0)
            keep = [w for w in e["want"] if start + w in wanted[e["id"]]]
            entries.append({"id": e["id"], "tokens": e["tokens"], "want": keep})
            fed[e["id"]] = start + len(e["tokens"])
        out.append({"step": step["step"], "entries": entries, "end": step["end"]})
    return out


def collect(session, steps: list[dict]) -> dict[str, torch.Tensor]:
    """Run ``steps`` through a ReplaySession; returns per request the logits of every
    position, in order (every step asks for all of its tokens)."""
    rows: dict[str, list[torch.Tensor]] = {}
    for step in steps:
        logits = session.run_step(step)
        if logits is None:
            assert not any(e["want"] for e in step["entries"])
            session.cache.check_invariants()
            continue
        r = 0
        for e in step["entries"]:
            for _ in e["want"]:
                rows.setdefault(e["id"], []).append(logits[r].clone())
                r += 1
        session.cache.check_invariants()
    return {rid: torch.stack(v) for rid, v in rows.items()}


def oracle_logits(cfg: dict, weights: dict, requests: dict[str, list[int]]) -> dict[str, torch.Tensor]:
    return {rid: plain_llama.logits_for(cfg, weights, toks) for rid, toks in requests.items()}


# Tolerances.  32-bit: the engine and the oracle add the same numbers in different orders;
# logits are O(1), so a few 1e-5 absolute is rounding and anything above it is a fault.
# bfloat16: activations are rounded to 8 bits of mantissa between the parts; with the peaked
# attention of `make_weights` that gives (measured with 32-bit arithmetic on bfloat16-rounded
# activations) up to 0.055 absolute, 0.032 relative RMS at the worst position and 0.012
# overall.  The bounds below leave a factor of about 2.5; a lost, misplaced or stale key
# moves a position's logits by tens of percent.
TOL = {"float32": dict(atol=3e-5, rtol=1e-5),
       "bfloat16": dict(atol=0.15, rtol=0.0, pos_rel_rms=0.08, rel_rms=0.03)}


# The largest differences every comparison has seen, per precision: printed at the end of a
# test run (tests/conftest.py), so that a drift towards the bounds shows before it fails.
ACHIEVED: dict[str, dict[str, float]] = {}


def _record(dtype: str, **values: float) -> None:
    seen = ACHIEVED.setdefault(dtype, {})
    for key, value in values.items():
        seen[key] = max(seen.get(key, 0.0), float(value))
    seen["comparisons"] = seen.get("comparisons", 0) + 1


def float32_tolerance(longest_sum: int, logit_scale: float) -> dict:
    """The 32-bit bound for any layer size.  Two correct 32-bit implementations add the same
    products in different orders; what they differ by grows with the square root of the longest
    sum (the largest inner dimension of a matrix product) and with the size of the logits:
    ``6 * 2^-23 * sqrt(longest_sum) * max|logit|``.  For the tiny configurations (sums of up to
    320 terms, logits up to 2.1) that is 2.7e-5, the fixed bound of ``TOL``; at hidden sizes of
    thousands it is some 1e-4.  Measured differences stay a factor of about ten below it at
    every size (3.7e-6 tiny, 6.2e-5 at the 8B layer shape), a misplaced key is 1e-2 and more."""
    return dict(atol=max(6 * 2.0 ** -23 * longest_sum ** 0.5 * max(logit_scale, 1.0), TOL["float32"]["atol"]),
                rtol=TOL["float32"]["rtol"])


def assert_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str, tol: dict | None = None) -> None:
    tol = tol or TOL[dtype]
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} != {tuple(want.shape)}"
    assert bool(torch.isfinite(got).all()), f"{what}: logits are not finite"
    got, want = got.double(), want.double()
    diff = (got - want).abs()
    bad = (diff > tol["atol"] + tol["rtol"] * want.abs()).any(dim=-1)
    pos_rel = diff.pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-12)
    _record(dtype, max_abs=diff.max() if diff.numel() else 0.0,
            max_pos_rel_rms=pos_rel.max() if pos_rel.numel() else 0.0)
    if "pos_rel_rms" in tol:
        bad = bad | (pos_rel > tol["pos_rel_rms"])
    if bool(bad.any()):
        idx = bad.nonzero().flatten()
        first = int(idx[0])
        raise AssertionError(
            f"{what}: {len(idx)} of {got.shape[0]} positions differ; first wrong position "
            f"{first} (max abs diff there {float(diff[first].max()):.3e}, overall "
            f"{float(diff.max()):.3e}, logits up to {float(want.abs().max()):.3f})")
    if "rel_rms" in tol:
        rel = float(diff.pow(2).mean().sqrt() / want.pow(2).mean().sqrt())
        _record(dtype, max_rel_rms=rel)
        assert rel < tol["rel_rms"], f"{what}: relative RMS error {rel:.3e} is too large"
