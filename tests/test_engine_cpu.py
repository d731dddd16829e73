"""The engine's logic without a GPU: scheduler, cache and step function together, on the plain
PyTorch stand-ins of the kernels, against the plain implementation's greedy generation.
Random workloads in the manner of the reference's tests/test_engine.py:207-251."""

from __future__ import annotations

import random

import pytest
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from tests import helpers as H
from tests import plain_llama
from tests.ref_ops import RefOps
from tests.tiny_configs import TINY_A, TINY_B


def _engine(cfg, weights, **kw):
    from inference_engine_b200.engine.llm_engine import LLMEngine
    from inference_engine_b200.engine.loading import model_from_tensors

    model, _ = model_from_tensors(cfg, weights, "float32", "cpu", cfg["max_position_embeddings"])
    return LLMEngine(model, None, kw.pop("stop_token_ids", ()), ops=RefOps(), debug_checks=True,
                     enable_cuda_graphs=False, **kw)


@pytest.mark.parametrize("seed", range(6))
def test_random_workloads_equal_plain_greedy(seed):
    _random_workload(seed)


@settings(max_examples=12, deadline=None, derandomize=True,
          suppress_health_check=[HealthCheck.too_slow])
@given(st.integers(min_value=6, max_value=2**31))
def test_random_workloads_drawn_by_hypothesis(seed):
    """The same property over seeds that Hypothesis draws (and shrinks, if one fails): sizes,
    pages, budgets, arrivals and an abort are all derived from the seed."""
    _random_workload(seed)


def _random_workload(seed):
    from inference_engine_b200 import SamplingParams

    rng = random.Random(seed)
    cfg = rng.choice([TINY_A, TINY_B])
    weights = H.make_weights(cfg, seed=seed)
    block_size = rng.choice([1, 2, 4, 8])
    max_tokens = rng.randint(2, 6)
    lengths = [rng.randint(1, 30) for _ in range(rng.randint(2, 5))]
    longest = max(lengths) + max_tokens
    num_blocks = -(-longest // block_size) + rng.randint(0, 2 * -(-longest // block_size))
    engine = _engine(cfg, weights, num_blocks=num_blocks, block_size=block_size,
                     max_num_seqs=rng.randint(1, 4), max_num_batched_tokens=rng.randint(4, 40),
                     enable_chunked_prefill=rng.random() < 0.8)
    prompts = {f"p{i}": H.random_tokens(cfg, n, 100 * seed + i) for i, n in enumerate(lengths)}
    params = SamplingParams(temperature=0, max_tokens=max_tokens)
    pending = list(prompts.items())
    got = {rid: [] for rid in prompts}
    aborted = None
    steps = 0
    while pending or engine.has_unfinished():
        while pending and rng.random() < 0.5:  # staggered arrivals
            rid, p = pending.pop(0)
            engine.add_request(rid, p, params)
        if aborted is None and steps == 3 and rng.random() < 0.5 and engine.scheduler.running:
            aborted = engine.scheduler.running[-1].request_id
            engine.abort(aborted)
        for out in engine.step():
            got[out.request_id].append(out.token_id)
        steps += 1
        assert steps < 2000
    for rid, prompt in prompts.items():
        if rid == aborted:
            continue
        assert got[rid] == plain_llama.greedy_generate(cfg, weights, prompt, max_tokens), rid
    assert engine.cache.num_free_pages == [num_blocks]
    assert engine.cache.slots.num_free == engine.cache.slots.num_slots


def test_step_records_and_snapshot():
    from inference_engine_b200 import SamplingParams

    cfg, weights = TINY_A, H.make_weights(TINY_A, seed=1)
    engine = _engine(cfg, weights, num_blocks=16, block_size=4, max_num_seqs=2, max_num_batched_tokens=8)
    engine.add_request("a", H.random_tokens(cfg, 11, 1), SamplingParams(temperature=0, max_tokens=3))
    outs = []
    while engine.has_unfinished():
        outs += engine.step()
    assert [o.completion_tokens for o in outs] == [1, 2, 3] and outs[-1].finish_reason == "length"
    assert outs[-1].prompt_tokens == 11 and outs[-1].finished and not outs[0].finished
    log = list(engine.step_log)
    assert [r["prefill_tokens"] for r in log] == [8, 3, 0, 0] and [r["decode_tokens"] for r in log] == [0, 0, 1, 1]
    snap = engine.snapshot()
    assert snap["totals"]["generated_tokens"] == 3 and snap["totals"]["finished_requests"] == 1
    assert snap["totals"]["prompt_tokens"] == 11 and snap["config"]["block_size"] == 4
    assert engine.step() == []


def test_logprobs_and_sampling_cutoffs():
    import torch

    from inference_engine_b200 import SamplingParams

    cfg, weights = TINY_B, H.make_weights(TINY_B, seed=2)
    engine = _engine(cfg, weights, num_blocks=32, block_size=8, max_num_seqs=2, max_num_batched_tokens=64)
    prompt = H.random_tokens(cfg, 12, 3)
    engine.add_request("a", prompt, SamplingParams(temperature=0, max_tokens=2, logprobs=True, top_logprobs=3))
    outs = []
    while engine.has_unfinished():
        outs += engine.step()
    lp = plain_llama.logits_for(cfg, weights, prompt)[-1].log_softmax(-1)
    assert outs[0].token_id == int(lp.argmax()) and abs(outs[0].logprob - float(lp.max())) < 1e-4
    assert [t for t, _ in outs[0].top_logprobs] == lp.topk(3).indices.tolist()
    # top_k = 1 at any temperature is greedy; a repetition penalty changes the choice rule
    sampled = engine.generate({"b": prompt}, SamplingParams(temperature=1.5, top_k=1, max_tokens=4, seed=1))["b"]
    assert sampled == plain_llama.greedy_generate(cfg, weights, prompt, 4)
    penal = engine.generate({"c": prompt}, SamplingParams(temperature=0, repetition_penalty=1.8, max_tokens=6))["c"]
    ids = list(prompt)
    for tok in penal:
        z = plain_llama.logits_for(cfg, weights, ids)[-1].clone()
        seen = torch.tensor(sorted(set(ids)))
        z[seen] = torch.where(z[seen] > 0, z[seen] / 1.8, z[seen] * 1.8)
        assert tok == int(z.argmax())
        ids.append(tok)


def test_stop_strings_need_a_tokenizer():
    from inference_engine_b200 import SamplingParams

    engine = _engine(TINY_A, H.make_weights(TINY_A), num_blocks=8, block_size=4, max_num_seqs=1,
                     max_num_batched_tokens=8)
    with pytest.raises(ValueError, match="tokenizer"):
        engine.add_request("a", [1, 2], SamplingParams(max_tokens=2, stop=("x",)))


def test_sampling_params_are_validated():
    from inference_engine_b200 import SamplingParams

    for bad in (dict(temperature=-1), dict(top_k=-1), dict(top_p=0.0), dict(top_p=1.5), dict(min_p=1.0),
                dict(repetition_penalty=0), dict(max_tokens=0), dict(top_logprobs=21),
                dict(top_logprobs=2, logprobs=False)):
        with pytest.raises(ValueError):
            SamplingParams(**bad)
    assert SamplingParams(temperature=0).greedy and not SamplingParams().greedy


def test_the_garbage_collector_is_off_while_a_step_is_captured():
    """An object the collector frees may own captured launch sequences or device memory; giving those
    back while a stream is capturing makes the capture invalid.  `graphs._capture` keeps the
    collector off until the capture has ended, also when the forward pass raises."""
    import contextlib
    import gc
    import types

    from inference_engine_b200.engine.graphs import _capture

    seen = []

    @contextlib.contextmanager
    def graph(_):
        seen.append(gc.isenabled())
        yield

    fake_torch = types.SimpleNamespace(cuda=types.SimpleNamespace(graph=graph))
    assert gc.isenabled()
    assert _capture(fake_torch, object(), lambda: (seen.append(gc.isenabled()), 7)[1]) == 7
    assert seen == [False, False] and gc.isenabled()

    def fails():
        raise RuntimeError("no")

    with pytest.raises(RuntimeError):
        _capture(fake_torch, object(), fails)
    assert gc.isenabled()
    gc.disable()
    try:  # (a caller that had it off gets it back off)
        _capture(fake_torch, object(), lambda: None)
        assert not gc.isenabled()
    finally:
        gc.enable()
