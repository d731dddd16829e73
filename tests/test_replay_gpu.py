"""Trace replay on the GPU against the plain implementation: every way of cutting the work,
in true 32-bit and in bfloat16, for tiny configurations that differ in every size."""

from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests import helpers as H
from tests.tiny_configs import PAGE_SIZE, TINY_A, TINY_B, TINY_C, TINY_D

pytestmark = pytest.mark.gpu
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}
LENGTHS = [70, 45, 33, 90, 20, 60]


@pytest.fixture(scope="module")
def cases(tmp_path_factory):
    out = {}
    for name, cfg in CONFIGS.items():
        weights = H.make_weights(cfg, seed=ord(name))
        folder = H.write_model_dir(tmp_path_factory.mktemp(f"tiny{name}"), cfg, weights)
        requests = {f"r{i}": H.random_tokens(cfg, n, 100 * ord(name) + i) for i, n in enumerate(LENGTHS)}
        out[name] = (cfg, folder, requests, H.oracle_logits(cfg, weights, requests))
    return out


def _session(folder, dtype, max_tokens, page_size):
    from inference_engine_b200.engine.replay import ReplaySession

    return ReplaySession(folder, dtype, max_tokens, device="cuda", page_size=page_size)


def _check(cases, name, dtype, steps, max_tokens):
    cfg, folder, requests, want = cases[name]
    session = _session(folder, dtype, max_tokens, PAGE_SIZE[name])
    got = H.collect(session, steps)
    for rid in requests:
        H.assert_close(got[rid], want[rid], dtype, f"tiny {name} {dtype} request {rid}")
    assert session.cache.num_free_pages == [p.num_pages for p in session.cache.pools]
    return got


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole(cases, name, dtype):
    _check(cases, name, dtype, H.trace_whole(cases[name][2]), 128)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_last_32_one_by_one(cases, name, dtype):
    _check(cases, name, dtype, H.trace_decode_tail(cases[name][2], 32), 128)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_of_changing_size(cases, name, dtype):
    _check(cases, name, dtype, H.trace_portions(cases[name][2]), 128)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("seed", [1, 2])
def test_mixed_with_pages_used_again(cases, name, dtype, seed):
    steps, peak = H.trace_mixed(cases[name][2], seed=seed)
    assert max(len(s["entries"]) for s in steps) >= 3
    assert peak < sum(H.round64(n) for n in LENGTHS)  # the pool is smaller than all requests
    _check(cases, name, dtype, steps, peak)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_float32_is_the_same_however_it_is_cut(cases, name):
    """In 32-bit a position's logits come out bit for bit the same whole, token by token, in
    portions and mixed with other requests: every reduction has a fixed order."""
    requests = cases[name][2]
    whole = _check(cases, name, "float32", H.trace_whole(requests), 128)
    steps, peak = H.trace_mixed(requests, seed=3)
    for other in (_check(cases, name, "float32", H.trace_decode_tail(requests, 32), 128),
                  _check(cases, name, "float32", H.trace_portions(requests), 128),
                  _check(cases, name, "float32", steps, peak)):
        for rid in requests:
            assert torch.equal(whole[rid], other[rid]), f"request {rid} depends on the cutting"


def test_first_tokens_and_single_token_requests(cases):
    """Position 0 alone, then the second token alone: the shortest contexts there are."""
    cfg, folder, requests, want = cases["B"]
    toks = requests["r0"]
    for dtype in ("float32", "bfloat16"):
        session = _session(folder, dtype, 64, PAGE_SIZE["B"])
        steps = [{"step": i, "entries": [{"id": "x", "tokens": [toks[i]], "want": [0]}], "end": []}
                 for i in range(10)]
        got = H.collect(session, steps)["x"]
        H.assert_close(got, want["r0"][:10], dtype, f"first tokens {dtype}")


def test_long_decoding(cases):
    """A long run of single tokens across many pages, from a two-token start."""
    cfg, folder, _, _ = cases["A"]
    from tests import plain_llama

    toks = H.random_tokens(cfg, 250, 77)
    weights = H.make_weights(cfg, seed=ord("A"))
    want = plain_llama.logits_for(cfg, weights, toks)
    for dtype in ("float32", "bfloat16"):
        session = _session(folder, dtype, 256, PAGE_SIZE["A"])
        steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:2], "want": [0, 1]}], "end": []}]
        steps += [{"step": i - 1, "entries": [{"id": "x", "tokens": [toks[i]], "want": [0]}], "end": []}
                  for i in range(2, len(toks))]
        H.assert_close(H.collect(session, steps)["x"], want, dtype, f"long decoding {dtype}")


def test_want_may_be_empty_and_requests_may_pause(cases):
    cfg, folder, requests, want = cases["A"]
    session = _session(folder, "float32", 192, PAGE_SIZE["A"])
    a, b = requests["r0"], requests["r1"]
    assert session.run_step({"step": 0, "entries": [{"id": "a", "tokens": a[:40], "want": []}], "end": []}) is None
    out = session.run_step({"step": 1, "entries": [{"id": "b", "tokens": b[:7], "want": [6]}], "end": []})
    H.assert_close(out, want["r1"][6:7], "float32", "b after a paused")
    out = session.run_step({"step": 2, "entries": [{"id": "a", "tokens": a[40:], "want": [len(a) - 41]},
                                                   {"id": "b", "tokens": b[7:9], "want": [0, 1]}],
                            "end": ["a", "b"]})
    H.assert_close(out[:1], want["r0"][-1:], "float32", "a resumed")
    H.assert_close(out[1:], want["r1"][7:9], "float32", "b beside a")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(cases, tmp_path, dtype):
    """The program itself: stdin lines in, `done <step>` lines and <step>.f32 files out."""
    cfg, folder, requests, want = cases["B"]
    steps, peak = H.trace_mixed(requests, seed=5)
    steps[3]["entries"][0]["want"] = []  # some steps want nothing from a request
    root = Path(__file__).resolve().parents[1]
    out_dir = tmp_path / "logits"
    proc = subprocess.run(
        [sys.executable, str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
         "--out", str(out_dir), "--max-tokens", str(peak), "--block-size", str(PAGE_SIZE["B"])],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
        timeout=600, env={**os.environ, "PYTHONPATH": ""})
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split("\n")[:-1] == [f"done {s['step']}" for s in steps]
    got = {rid: [] for rid in requests}
    places = {rid: [] for rid in requests}
    fed = {rid: 0 for rid in requests}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        path = out_dir / f"{s['step']}.f32"
        if wanted == 0:
            assert not path.exists()
        else:
            assert path.stat().st_size == wanted * cfg["vocab_size"] * 4
            arr = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(wanted, cfg["vocab_size"]).copy())
            r = 0
            for e in s["entries"]:
                for w in e["want"]:
                    got[e["id"]].append(arr[r])
                    places[e["id"]].append(fed[e["id"]] + w)
                    r += 1
        for e in s["entries"]:
            fed[e["id"]] += len(e["tokens"])
    for rid in requests:
        H.assert_close(torch.stack(got[rid]), want[rid][places[rid]], dtype, f"trace_run {dtype} {rid}")
