"""Short steps that hold prompt portions, replayed as captured launch sequences
(`engine/graphs.py: MixedGraphs`), against the plain implementation and against the same steps
launched eagerly: whole prompts, portions of changing size down to two tokens, portions beside
decoded tokens of other requests with pages that are used again, in true 32-bit and in bfloat16.

A capture is made for bounds (tokens, sequences, wanted rows, block-table stride), not for a step:
the same launch sequence must serve every step that fits, so every trace below replays each of its
few captures for many different cuttings."""

from __future__ import annotations

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


def _session(folder, dtype, max_tokens, page_size, captured: bool):
    """A replay session; with `captured`, every step that holds a portion and fits a capture goes
    through it (steps of single tokens stay eager here: the decode captures have their own tests)."""
    from inference_engine_b200.engine.graphs import DecodeGraphs, MixedGraphs
    from inference_engine_b200.engine.replay import ReplaySession

    session = ReplaySession(folder, dtype, max_tokens, device="cuda", page_size=page_size)
    session.mixed = None
    if captured:
        width = max(64, -(-max_tokens // page_size))
        session.mixed = MixedGraphs(DecodeGraphs(session.runner, 256, width))
        eager = session.runner.step

        def step(entries):
            if session.mixed.can_run(entries):
                return session.mixed.run(entries)
            assert all(len(e.tokens) == 1 for e in entries) or sum(len(e.tokens) for e in entries) > 1024
            return eager(entries)

        session.runner.step = step
    return session


def _run(cases, name, dtype, steps, max_tokens, captured=True):
    cfg, folder, requests, want = cases[name]
    session = _session(folder, dtype, max_tokens, PAGE_SIZE[name], captured)
    got = H.collect(session, steps)
    for rid in requests:
        H.assert_close(got[rid], want[rid], dtype, f"tiny {name} {dtype} request {rid}, captured steps")
    assert session.cache.num_free_pages == [p.num_pages for p in session.cache.pools]
    return got, session


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompts_and_portions(cases, name, dtype):
    requests = cases[name][2]
    whole, session = _run(cases, name, dtype, H.trace_whole(requests), 128)
    assert session.mixed.replays == len(requests)
    assert len(session.mixed._graphs) < len(requests)  # (prompts of like length share a launch sequence)
    portions, session = _run(cases, name, dtype, H.trace_portions(requests), 128)
    assert session.mixed.replays > 3 * len(requests)
    if dtype == "float32":  # every reduction has a fixed order, whatever the launch is padded to
        eager, _ = _run(cases, name, dtype, H.trace_portions(requests), 128, captured=False)
        for rid in requests:
            assert torch.equal(whole[rid], portions[rid]) and torch.equal(eager[rid], portions[rid])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("seed", [1, 2])
def test_portions_beside_decoded_tokens_with_pages_used_again(cases, name, dtype, seed):
    steps, peak = H.trace_mixed(cases[name][2], seed=seed)
    assert max(len(s["entries"]) for s in steps) >= 3
    got, session = _run(cases, name, dtype, steps, peak)
    mixed_steps = sum(1 for s in steps if any(len(e["tokens"]) > 1 for e in s["entries"]))
    assert session.mixed.replays == mixed_steps and mixed_steps > 10
    assert len(session.mixed._graphs) < mixed_steps  # captures are shared among steps


def test_a_step_may_want_nothing_and_a_long_one_runs_eagerly(cases):
    cfg, folder, requests, want = cases["A"]
    session = _session(folder, "bfloat16", 1408, PAGE_SIZE["A"], captured=True)
    a, b = requests["r0"], requests["r1"]
    assert session.run_step({"step": 0, "entries": [{"id": "a", "tokens": a[:40], "want": []}], "end": []}) is None
    assert session.mixed.replays == 1
    out = session.run_step({"step": 1, "entries": [{"id": "a", "tokens": a[40:], "want": [len(a) - 41]},
                                                   {"id": "b", "tokens": b[:9], "want": [7, 8]}], "end": ["a"]})
    H.assert_close(out[:1], want["r0"][-1:], "bfloat16", "a resumed in a captured step")
    H.assert_close(out[1:], want["r1"][7:9], "bfloat16", "b beside a")
    assert session.mixed.replays == 2
    # more tokens than the largest capture holds: launched eagerly
    long = H.random_tokens(cfg, 1100, 5)
    out = session.run_step({"step": 2, "entries": [{"id": "c", "tokens": long, "want": [1099]}], "end": ["c"]})
    assert out is not None and session.mixed.replays == 2
    session.ops.check_errors()


def test_the_engine_captures_short_steps_by_default():
    """Generation through the engine: prompts arrive while others decode, every step is a captured
    one (decode steps and steps with portions), and every token is the plain implementation's."""
    from inference_engine_b200 import SamplingParams
    from inference_engine_b200.engine.llm_engine import LLMEngine
    from inference_engine_b200.engine.loading import model_from_tensors
    from tests.test_engine_gpu import _check_greedy

    cfg, weights = TINY_B, H.make_weights(TINY_B, seed=31)
    model, _ = model_from_tensors(cfg, weights, "bfloat16", "cuda", cfg["max_position_embeddings"])
    engine = LLMEngine(model, None, (), num_blocks=60, block_size=8, max_num_seqs=4, max_num_batched_tokens=32,
                       debug_checks=True)
    assert engine.mixed_graphs is not None
    prompts = {f"p{i}": H.random_tokens(cfg, n, 300 + i) for i, n in enumerate([50, 7, 23, 41, 3, 30])}
    got = engine.generate(prompts, SamplingParams(temperature=0, max_tokens=12))
    assert engine.mixed_graphs.replays >= 3 and engine.graphs.replays > 0
    for rid, prompt in prompts.items():
        assert len(got[rid]) == 12
        _check_greedy(cfg, weights, prompt, got[rid], "bfloat16")
    eager = LLMEngine(model, None, (), num_blocks=60, block_size=8, max_num_seqs=4, max_num_batched_tokens=32,
                      enable_mixed_graphs=False)
    assert eager.mixed_graphs is None and eager.graphs is not None


def test_warm_up_captures_ahead_of_the_first_request():
    """`LLMEngine.warm_up()`: the decode buckets and the token buckets are captured on an idle engine,
    every page comes back, and a generation afterwards replays those captures instead of making its own."""
    from inference_engine_b200 import SamplingParams
    from inference_engine_b200.engine.llm_engine import LLMEngine
    from inference_engine_b200.engine.loading import model_from_tensors
    from tests.test_engine_gpu import _check_greedy

    cfg, weights = TINY_B, H.make_weights(TINY_B, seed=32)
    model, _ = model_from_tensors(cfg, weights, "bfloat16", "cuda", cfg["max_position_embeddings"])
    engine = LLMEngine(model, None, (), num_blocks=60, block_size=8, max_num_seqs=4, max_num_batched_tokens=48,
                       debug_checks=True)
    captured = engine.warm_up()
    assert captured == len(engine.graphs.buckets) + len([t for t in engine.mixed_graphs.token_buckets if t >= 2])
    assert engine.cache.num_free_pages == [60] and not engine.has_unfinished()
    decode_keys, mixed_keys = set(engine.graphs._graphs), set(engine.mixed_graphs._graphs)
    prompts = {f"p{i}": H.random_tokens(cfg, n, 400 + i) for i, n in enumerate([30, 7, 2])}
    got = engine.generate(prompts, SamplingParams(temperature=0, max_tokens=8))
    for rid, prompt in prompts.items():
        _check_greedy(cfg, weights, prompt, got[rid], "bfloat16")
    assert set(engine.graphs._graphs) == decode_keys  # (decode steps of 1 to 3 requests: buckets 1, 2, 4)
    assert len(set(engine.mixed_graphs._graphs) - mixed_keys) <= 1  # (at most the step that needed a larger sequence bucket)
    with pytest.raises(RuntimeError):
        engine.add_request("x", [1, 2, 3], SamplingParams(temperature=0, max_tokens=4))
        engine.warm_up()
