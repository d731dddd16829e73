"""New parts from outside the package: a mixer with state of its own, a routed feed-forward,
an additive position encoding, a layer that runs twice, a run that reads another run's cache
and a windowed cache group whose pages are given back.  Registered, built, loaded and stepped
without a change to the framework's files; compared with a whole-sequence oracle under every
way of cutting the work."""

from __future__ import annotations

import pytest
import torch

from tests import helpers as H
from tests import toy_parts as T


def _session(tmp_path, device, ops, max_tokens, page_size=4):
    from inference_engine_b200.engine.replay import ReplaySession

    weights = T.toy_weights(seed=2)
    folder = H.write_model_dir(tmp_path / "toy", T.TOY_CONFIG, weights)
    return ReplaySession(folder, "float32", max_tokens, device=device, ops=ops, page_size=page_size), weights


def _run_all_modes(tmp_path, device, ops):
    T.register_toys()
    requests = {f"r{i}": H.random_tokens(T.TOY_CONFIG, n, 300 + i) for i, n in enumerate([50, 21, 37, 64, 9])}
    steps, peak = H.trace_mixed(requests, seed=4, tail=6, max_portion=14)
    weights = T.toy_weights(seed=2)
    want = {rid: T.plain_toy_logits(weights, toks) for rid, toks in requests.items()}
    for name, (trace, max_tokens) in {"whole": (H.trace_whole(requests), 128),
                                      "tail": (H.trace_decode_tail(requests, 12), 128),
                                      "portions": (H.trace_portions(requests, (5, 2, 13, 3, 2)), 128),
                                      "mixed": (steps, peak)}.items():
        session, _ = _session(tmp_path, device, ops, max_tokens)
        model = session.model
        assert [type(b.mixer).__name__ for b in model.blocks] == ["PagedAttention", "ToyStateMixer", "PagedAttention"]
        # two paged groups (all positions; a window of 11) and one state group with two runs
        assert [(g.num_layers, g.window) for g in model.paged_groups] == [(1, None), (1, 11)]
        assert [(g.num_layers, g.shape) for g in model.state_groups] == [(2, (24,))]
        assert model.bindings[4].writes is False and model.bindings[4].slot == model.bindings[0].slot
        got = H.collect(session, trace)
        for rid in requests:
            H.assert_close(got[rid], want[rid], "float32", f"toy {name} {rid}")
        assert session.cache.num_free_pages == [p.num_pages for p in session.cache.pools]
        assert session.cache.slots.num_free == session.cache.slots.num_slots


def test_toy_architecture_on_reference_ops(tmp_path):
    from tests.ref_ops import RefOps

    _run_all_modes(tmp_path, "cpu", RefOps())


@pytest.mark.gpu
def test_toy_architecture_on_the_gpu(tmp_path):
    from inference_engine_b200.kernels import get_ops

    _run_all_modes(tmp_path, "cuda", get_ops("cuda"))


def test_window_pages_are_given_back_while_decoding(tmp_path):
    from tests.ref_ops import RefOps

    T.register_toys()
    session, weights = _session(tmp_path, "cpu", RefOps(), 64)
    toks = H.random_tokens(T.TOY_CONFIG, 60, 1)
    session.run_step({"step": 0, "entries": [{"id": "a", "tokens": toks[:40], "want": []}], "end": []})
    full, windowed = (len([p for p in session.cache.table(g, "a") if p >= 0]) for g in (0, 1))
    assert full == 10 and windowed == 3  # window 11 over pages of 4: positions 30..39 -> 3 pages
    for i in range(40, 60):
        session.run_step({"step": i, "entries": [{"id": "a", "tokens": [toks[i]], "want": []}], "end": []})
        held = len([p for p in session.cache.table(1, "a") if p >= 0])
        assert held <= 4
    session.cache.check_invariants()


def test_an_unknown_kind_is_refused_with_the_known_ones():
    from inference_engine_b200.config.spec import PartSpec
    from inference_engine_b200.parts import BuildEnv, build_part

    with pytest.raises(ValueError, match="no mixer of kind 'nope'.*paged_attention"):
        build_part("mixer", PartSpec("nope"), BuildEnv(8, "float32", 8, {}))


# --- two attention groups of different head size, one windowed; captured and launched ahead -----


def _two_attentions_folder(tmp_path):
    T.register_toys()
    weights = T.two_attentions_weights(seed=5)
    return H.write_model_dir(tmp_path / "two", T.TWO_ATTENTIONS_CONFIG, weights), weights


def _two_attentions_replay(tmp_path, device, ops, dtype):
    from inference_engine_b200.engine.replay import ReplaySession

    folder, weights = _two_attentions_folder(tmp_path)
    cfg = T.TWO_ATTENTIONS_CONFIG
    requests = {f"r{i}": H.random_tokens(cfg, n, 500 + i) for i, n in enumerate([70, 23, 41, 64, 9])}
    want = {rid: T.plain_two_attentions_logits(weights, toks) for rid, toks in requests.items()}
    mixed, peak = H.trace_mixed(requests, seed=6, tail=8, max_portion=20)
    for name, (trace, max_tokens) in {"whole": (H.trace_whole(requests), 128),
                                      "tail": (H.trace_decode_tail(requests, 20), 128),
                                      "portions": (H.trace_portions(requests, (5, 2, 19, 3, 2, 30)), 128),
                                      "mixed": (mixed, peak)}.items():
        session = ReplaySession(folder, dtype, max_tokens, device=device, ops=ops, page_size=4)
        groups = session.model.paged_groups
        assert [(g.num_layers, g.num_kv_heads, g.head_dim, g.window) for g in groups] == [(2, 2, 16, None), (1, 1, 32, 11)]
        got = H.collect(session, trace)
        for rid in requests:
            H.assert_close(got[rid], want[rid], dtype, f"two attentions {dtype} {name} {rid}")
        assert session.cache.num_free_pages == [p.num_pages for p in session.cache.pools]


def test_two_attention_groups_on_reference_ops(tmp_path):
    from tests.ref_ops import RefOps

    _two_attentions_replay(tmp_path, "cpu", RefOps(), "float32")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_attention_groups_on_the_gpu(tmp_path, dtype):
    from inference_engine_b200.kernels import get_ops

    _two_attentions_replay(tmp_path, "cuda", get_ops("cuda"), dtype)


def test_engine_info_asks_the_architecture(tmp_path, capsys):
    """`engine info` on a folder of an architecture registered from outside the package, which
    reports no footprint of its own: the model is put together and counted."""
    from inference_engine_b200.cli import main

    folder, weights = _two_attentions_folder(tmp_path)
    assert main(["info", "--model", str(folder), "--gpu-mem", "80"]) == 0
    text = capsys.readouterr().out
    params = sum(t.numel() for t in weights.values())
    assert "ToyTwoAttentionsForTests" in text and f"{params / 1e9:.3f} B" in text
    # keys and values per token: the wide layer runs twice (2 x 2 heads x 16), the narrow once (1 x 32)
    assert f"{2 * (2 * 2 * 16 + 32) * 2 / 1024:.1f} KiB" in text and "KV tokens fit" in text


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_windowed_model_decodes_in_captured_steps_launched_ahead(tmp_path, dtype):
    """A model with a windowed cache group decodes in captured steps that are launched before
    the previous step's tokens were fetched.  A request that hits a stop id, one that is aborted
    and one that reaches its limit end while such a step is already running for them: their
    pages (also those the window gave back earlier) are returned once, the others' tokens are
    those of an engine that launches nothing ahead."""
    from inference_engine_b200 import SamplingParams
    from inference_engine_b200.engine.llm_engine import LLMEngine
    from inference_engine_b200.engine.loading import load_model

    folder, weights = _two_attentions_folder(tmp_path)
    cfg = T.TWO_ATTENTIONS_CONFIG
    prompts = [H.random_tokens(cfg, n, 700 + i) for i, n in enumerate([5, 30, 17, 44])]
    limits = [40, 13, 40, 25]

    def run(ahead, stop_ids):
        model, _ = load_model(folder, dtype, "cuda", max_positions=256)
        engine = LLMEngine(model, None, stop_ids, num_blocks=96, block_size=4, max_num_seqs=4,
                           max_num_batched_tokens=32, debug_checks=True)
        assert engine.graphs is not None  # no state slots: captured by default
        engine.launch_ahead = ahead
        for i, prompt in enumerate(prompts):
            engine.add_request(f"r{i}", prompt, SamplingParams(temperature=0, max_tokens=limits[i]))
        got, steps, ahead_steps = {}, 0, 0
        while engine.has_unfinished():
            steps += 1
            if steps == 12:
                assert engine.abort("r2")
            ahead_steps += engine._ahead is not None
            for out in engine.step():
                got.setdefault(out.request_id, []).append((out.token_id, out.finish_reason))
        assert engine._ahead is None
        assert engine.cache.num_free_pages == [96, 96]
        engine.cache.check_invariants()
        return got, ahead_steps

    free_run, _ = run(False, ())
    stop = free_run["r0"][15][0]  # a token the longest request produces in mid-course
    want, none_ahead = run(False, (stop,))
    got, ahead_steps = run(True, (stop,))
    assert none_ahead == 0 and ahead_steps > 8
    assert got == want
    assert got["r0"][-1][1] == "stop" and len(got["r0"]) < limits[0]
    # and the tokens are the plain implementation's
    ids = list(prompts[3])
    for token, _ in got["r3"]:
        logits = T.plain_two_attentions_logits(weights, ids)[-1]
        best = int(logits.argmax())
        assert token == best or (dtype == "bfloat16" and float(logits[best] - logits[token]) < 0.1)
        ids.append(token)


def test_abort_drops_a_step_that_runs_ahead_for_nobody():
    """What `abort` does when the step running ahead was for the aborted requests only; and the
    cache manager's answer for a request it no longer knows."""
    from inference_engine_b200.cache import CacheManager, PagedGroupSpec

    cache = CacheManager([PagedGroupSpec(1, 1, 8, window=6)], [], 8, 4, 2)
    cache.add_request("a")
    cache.grow("a", 0, 13)
    assert cache.release_behind_window("a", 13) == 2
    cache.free("a")
    assert cache.release_behind_window("a", 14) == 0  # it ended while a step ran ahead for it
    cache.check_invariants()
