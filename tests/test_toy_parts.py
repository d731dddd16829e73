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
