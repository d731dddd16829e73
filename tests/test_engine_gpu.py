"""The engine end to end on the GPU: generation through the Python entry points against the
plain implementation, captured decode steps against eager ones, preemption with few pages,
seeded sampling that does not depend on the batch."""

from __future__ import annotations

import pytest
import torch

from tests import helpers as H
from tests import plain_llama
from tests.tiny_configs import PAGE_SIZE, TINY_A, TINY_B

pytestmark = pytest.mark.gpu


def _engine(cfg, weights, dtype, **kw):
    from inference_engine_b200.engine.llm_engine import LLMEngine
    from inference_engine_b200.engine.loading import model_from_tensors

    model, _ = model_from_tensors(cfg, weights, dtype, "cuda", cfg["max_position_embeddings"])
    kw.setdefault("debug_checks", True)
    return LLMEngine(model, None, kw.pop("stop_token_ids", ()), **kw)


def _random_model_weights(cfg, seed):
    """The tensors `LLMEngine.from_random(cfg, seed)` draws, as the plain implementation wants them."""
    from inference_engine_b200.config import build_model_spec, config_from_dict
    from inference_engine_b200.engine.model import declared_weights
    from inference_engine_b200.weights.random_weights import random_tensors

    decl = declared_weights(build_model_spec(config_from_dict(cfg)))
    # (drawn on the device, as the engine draws them: the CPU's generator gives other numbers)
    return {n: t.cpu() for n, t in random_tensors(decl, seed, 0.02, torch.bfloat16, "cuda").items()}


def _check_greedy(cfg, weights, prompt, got, dtype):
    """Every produced token is the plain implementation's argmax given the same prefix; in
    bfloat16 a token within a small logit gap of the argmax also counts (near ties flip)."""
    ids = list(prompt)
    for i, token in enumerate(got):
        logits = plain_llama.logits_for(cfg, weights, ids)[-1]
        best = int(logits.argmax())
        if token != best:
            gap = float(logits[best] - logits[token])
            assert dtype == "bfloat16" and gap < 0.1, (
                f"token {i}: engine chose {token}, plain chose {best} (gap {gap:.4f})")
        ids.append(token)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,cfg,lengths,max_tokens", [
    ("A", TINY_A, [5, 17, 33], 8), ("B", TINY_B, [1, 9, 40, 70], 12)])
def test_greedy_generation_matches_plain(name, cfg, lengths, max_tokens, dtype):
    from inference_engine_b200 import SamplingParams

    weights = H.make_weights(cfg, seed=3)
    engine = _engine(cfg, weights, dtype, num_blocks=64, block_size=PAGE_SIZE[name],
                     max_num_seqs=4, max_num_batched_tokens=24)
    prompts = {f"p{i}": H.random_tokens(cfg, n, 40 + i) for i, n in enumerate(lengths)}
    out = engine.generate(prompts, SamplingParams(temperature=0, max_tokens=max_tokens))
    for rid, prompt in prompts.items():
        assert len(out[rid]) == max_tokens
        _check_greedy(cfg, weights, prompt, out[rid], dtype)
    assert engine.cache.num_free_pages == [64]
    assert not engine.has_unfinished()


def test_generate_entry_point_and_stop_ids():
    """`generate(model, tokenizer, prompts, params, stop_token_ids)` yields one output per
    sequence and step; a stop id is returned as the last token with reason "stop"."""
    from inference_engine_b200 import SamplingParams, generate
    from inference_engine_b200.engine.loading import model_from_tensors

    cfg, weights = TINY_A, H.make_weights(TINY_A, seed=4)
    model, _ = model_from_tensors(cfg, weights, "float32", "cuda", 256)
    prompts = [H.random_tokens(cfg, n, 50 + n) for n in (6, 21)]
    free_run = [plain_llama.greedy_generate(cfg, weights, p, 10) for p in prompts]
    stop = free_run[1][4]
    outs = list(generate(model, None, prompts, SamplingParams(temperature=0, max_tokens=10), (stop,)))
    for i, p in enumerate(prompts):
        mine = [o for o in outs if o.seq_index == i]
        want = plain_llama.greedy_generate(cfg, weights, p, 10, stop_ids=(stop,))
        assert [o.token_id for o in mine] == want
        assert mine[-1].finished and mine[-1].finish_reason == ("stop" if want[-1] == stop else "length")
        assert all(not o.finished for o in mine[:-1])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_decode_steps_equal_eager_ones(dtype):
    from inference_engine_b200 import SamplingParams

    cfg, weights = TINY_B, H.make_weights(TINY_B, seed=5)
    prompts = {f"p{i}": H.random_tokens(cfg, n, 60 + i) for i, n in enumerate([3, 30, 11])}
    outs = []
    for graphs in (False, True):
        engine = _engine(cfg, weights, dtype, num_blocks=40, block_size=8, max_num_seqs=4,
                         max_num_batched_tokens=64, enable_cuda_graphs=graphs)
        outs.append(engine.generate(prompts, SamplingParams(temperature=0, max_tokens=20)))
        if graphs:
            assert engine.graphs.replays >= 15
    assert outs[0] == outs[1]


def test_preemption_with_few_pages_gives_the_same_tokens():
    """So few pages that running requests are preempted and prefilled again: the tokens are
    those of each request alone (engine/runtime tests of the reference: test_engine.py:92-97)."""
    from inference_engine_b200 import SamplingParams

    cfg, weights = TINY_A, H.make_weights(TINY_A, seed=6)
    prompts = {f"p{i}": H.random_tokens(cfg, n, 70 + i) for i, n in enumerate([20, 33, 14, 27])}
    params = SamplingParams(temperature=0, max_tokens=24)
    roomy = _engine(cfg, weights, "float32", num_blocks=64, block_size=4, max_num_seqs=4,
                    max_num_batched_tokens=16)
    want = roomy.generate(prompts, params)
    tight = _engine(cfg, weights, "float32", num_blocks=24, block_size=4, max_num_seqs=4,
                    max_num_batched_tokens=16)
    got = tight.generate(prompts, params)
    assert tight.scheduler.num_preemptions > 0
    assert got == want
    assert tight.cache.num_free_pages == [24]


def test_preemption_in_bfloat16_with_captured_steps():
    """The same with the serving kernels and captured decode steps: requests that lose their pages
    are prefilled again (through the prefill kernels, where the first time they decoded), so a
    token may differ at a near tie; every token is the plain implementation's choice given the
    tokens before it, or within a small gap of it, and every page comes back."""
    from inference_engine_b200 import SamplingParams

    cfg, weights = TINY_B, H.make_weights(TINY_B, seed=16)
    prompts = {f"p{i}": H.random_tokens(cfg, n, 170 + i) for i, n in enumerate([20, 33, 14, 27, 9])}
    params = SamplingParams(temperature=0, max_tokens=24)
    tight = _engine(cfg, weights, "bfloat16", num_blocks=14, block_size=8, max_num_seqs=4,
                    max_num_batched_tokens=24, enable_cuda_graphs=True)
    got = tight.generate(prompts, params)
    assert tight.scheduler.num_preemptions > 0 and tight.graphs.replays > 0
    for rid, prompt in prompts.items():
        assert len(got[rid]) == 24
        _check_greedy(cfg, weights, prompt, got[rid], "bfloat16")
    assert tight.cache.num_free_pages == [14]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_launched_ahead_give_the_same_tokens(dtype):
    """A decode step may start on the tokens the device is still sampling, before the host has
    seen them.  Requests that stop at a stop id or at their own limit, one that is aborted and
    one that arrives late, with greedy and with seeded sampling: the tokens and the reasons are
    those of an engine that fetches every token before it launches the next step."""
    from inference_engine_b200 import SamplingParams

    cfg, weights = TINY_B, H.make_weights(TINY_B, seed=11)
    prompts = [H.random_tokens(cfg, n, 90 + i) for i, n in enumerate([3, 21, 40, 9, 17])]
    limits = [30, 11, 24, 30, 16]

    def run(ahead: bool, stop_ids):
        engine = _engine(cfg, weights, dtype, num_blocks=64, block_size=8, max_num_seqs=4,
                         max_num_batched_tokens=24, stop_token_ids=stop_ids)
        engine.launch_ahead = ahead
        for i in range(4):
            sampling = dict(temperature=0) if i % 2 == 0 else dict(temperature=0.7, seed=50 + i, top_k=20)
            engine.add_request(f"r{i}", prompts[i], SamplingParams(max_tokens=limits[i], **sampling))
        got, steps, ahead_steps = {}, 0, 0
        while engine.has_unfinished():
            steps += 1
            if steps == 9:
                assert engine.abort("r3")
            if steps == 14:
                engine.add_request("r4", prompts[4], SamplingParams(temperature=0, max_tokens=limits[4]))
            ahead_steps += engine._ahead is not None
            for out in engine.step():
                got.setdefault(out.request_id, []).append((out.token_id, out.finished, out.finish_reason))
        assert engine.cache.num_free_pages == [64]
        return got, ahead_steps

    plain, none_ahead = run(False, ())
    assert none_ahead == 0
    # a stop id that the longest greedy request produces in mid-course
    stop = plain["r0"][12][0]
    want, _ = run(False, (stop,))
    got, ahead_steps = run(True, (stop,))
    assert ahead_steps > 10
    assert got == want
    assert any(reason == "stop" for _, _, reason in (v[-1] for v in got.values()))
    assert len(got["r3"]) < limits[3] and not got["r3"][-1][1]  # aborted
    assert len(got["r4"]) == limits[4] or got["r4"][-1][2] == "stop"


def test_seeded_sampling_does_not_depend_on_the_batch():
    from inference_engine_b200 import SamplingParams

    cfg, weights = TINY_B, H.make_weights(TINY_B, seed=7)
    prompts = {f"p{i}": H.random_tokens(cfg, n, 80 + i) for i, n in enumerate([1, 9, 40, 70])}
    params = SamplingParams(temperature=0.8, max_tokens=12, seed=1234)
    engine = _engine(cfg, weights, "float32", num_blocks=64, block_size=8, max_num_seqs=4,
                     max_num_batched_tokens=24)
    together = engine.generate(prompts, params)
    for rid, prompt in prompts.items():
        assert engine.generate({rid: prompt}, params)[rid] == together[rid]
    assert len({tuple(v) for v in together.values()}) > 1
    other = engine.generate(prompts, SamplingParams(temperature=0.8, max_tokens=12, seed=99))
    assert other != together


def test_requests_that_cannot_fit_are_refused():
    from inference_engine_b200 import SamplingParams

    cfg, weights = TINY_A, H.make_weights(TINY_A, seed=8)
    engine = _engine(cfg, weights, "float32", num_blocks=4, block_size=16, max_num_seqs=2,
                     max_num_batched_tokens=16)
    with pytest.raises(ValueError, match="exceeds"):
        engine.add_request("big", [1] * 60, SamplingParams(max_tokens=10))
    with pytest.raises(ValueError, match="at least one token"):
        engine.add_request("empty", [], SamplingParams(max_tokens=1))
    engine.add_request("ok", [1, 2, 3], SamplingParams(max_tokens=2))
    with pytest.raises(ValueError, match="duplicate"):
        engine.add_request("ok", [1], SamplingParams(max_tokens=2))
    with pytest.raises(ValueError, match="vocabulary"):
        engine.add_request("bad", [cfg["vocab_size"]], SamplingParams(max_tokens=2))
    assert engine.abort("ok") and not engine.abort("ok")
    assert engine.cache.num_free_pages == [4]


def test_a_kernel_report_reaches_the_host_with_the_tokens():
    """Without `debug_checks` too: the kernels' error word travels with every step's tokens, and
    a step whose kernels reported a bad index (or a wait that ran out) raises instead of
    handing out tokens; the word is cleared for the next report."""
    from inference_engine_b200 import SamplingParams
    from inference_engine_b200.kernels import KernelError

    cfg, weights = TINY_A, H.make_weights(TINY_A, seed=9)
    engine = _engine(cfg, weights, "bfloat16", num_blocks=16, block_size=16, max_num_seqs=2,
                     max_num_batched_tokens=32, debug_checks=False)
    engine.add_request("a", H.random_tokens(cfg, 9, 1), SamplingParams(temperature=0, max_tokens=8))
    assert len(engine.step()) == 1  # prefill and first token: nothing reported
    engine.ops.err.copy_(torch.tensor([2, 77, 3, 0], dtype=torch.int32))  # as a kernel would leave it
    with pytest.raises(KernelError, match="page or slot outside the cache.*77"):
        while engine.has_unfinished():
            engine.step()
    torch.cuda.synchronize()
    assert engine.ops.err.tolist() == [0, 0, 0, 0]
    engine.abort("a")


def test_smoke_entry():
    import __graft_entry__

    __graft_entry__.smoke()


@pytest.mark.gpu
def test_a_long_request_among_short_ones_decodes_the_same_with_either_attention_launch(monkeypatch):
    """The decode attention that deals key tiles by length (for contexts that differ much;
    captured separately) gives the tokens of the launch that deals them by request."""
    from inference_engine_b200 import SamplingParams
    from inference_engine_b200.engine.llm_engine import LLMEngine

    g = torch.Generator().manual_seed(5)
    vocab = TINY_A["vocab_size"]
    prompts = {"long": torch.randint(0, vocab, (900,), generator=g).tolist()}
    for i in range(5):
        prompts[f"short{i}"] = torch.randint(0, vocab, (7 + 3 * i,), generator=g).tolist()
    params = SamplingParams(temperature=0, max_tokens=12)
    results = {}
    for mode in ("1", "0"):
        cfg = dict(TINY_A, max_position_embeddings=2048)
        eng = LLMEngine.from_random(cfg, seed=3, dtype="bfloat16", device="cuda", max_model_len=1024,
                                    num_blocks=160, block_size=8, max_num_seqs=8, enable_cuda_graphs=True)
        monkeypatch.setattr(eng.ops, "decode_balanced", mode)
        before = eng.ops.balanced_launches
        results[mode] = eng.generate(prompts, params)
        assert (eng.ops.balanced_launches > before) == (mode == "1")
        assert all(key[1] == ((mode == "1"),) for key in eng.graphs._graphs) and eng.graphs._graphs
        eng.ops.check_errors()
    # Each launch's tokens are the plain implementation's choices (or within a small gap of them:
    # a near-tie may flip between summation orders), request by request.
    weights = _random_model_weights(cfg, seed=3)
    for mode in ("1", "0"):
        for rid, prompt in prompts.items():
            _check_greedy(cfg, weights, prompt, results[mode][rid], "bfloat16")
    # left to itself the engine deals by length only where that pays
    monkeypatch.setattr(eng.ops, "decode_balanced", "auto")
    assert eng.ops.decode_by_length([32768] + [256] * 31, 8)
    assert eng.ops.decode_by_length([8000] + [500] * 7, 8)
    assert not eng.ops.decode_by_length([1024] * 8, 8)
    assert not eng.ops.decode_by_length([2304] * 32, 8)
