"""The plain implementation itself: each part against a direct evaluation of its formula, and
the whole against outputs of the reference's own model code (tests/golden/)."""

from __future__ import annotations

import math
from pathlib import Path

import numpy as np
import pytest
import torch

from tests import helpers, plain_llama as P
from tests.tiny_configs import TINY_A, TINY_B, TINY_C

GOLDEN = Path(__file__).parent / "golden"


@pytest.mark.parametrize("name,cfg", [("A", TINY_A), ("B", TINY_B), ("C", TINY_C)])
def test_against_the_reference_models_outputs(name, cfg):
    data = np.load(GOLDEN / f"golden_{name}.npz")
    weights = helpers.make_weights(cfg, seed=ord(name))
    logits = P.logits_for(cfg, weights, data["token_ids"].tolist())
    rows = data["rows"].tolist()
    torch.testing.assert_close(logits[rows], torch.from_numpy(data["row_logits"]), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(logits[:, ::7], torch.from_numpy(data["strided_logits"]), atol=1e-5, rtol=1e-5)


def test_rms_norm_formula():
    x = torch.randn(5, 96) * 3
    w = torch.randn(96)
    out = P.rms_norm(x, w, 1e-6)
    for r in range(5):
        ms = sum(float(v) ** 2 for v in x[r]) / 96
        want = w * x[r] / math.sqrt(ms + 1e-6)
        torch.testing.assert_close(out[r], want, atol=1e-5, rtol=1e-5)


def test_rope_frequencies_plain_and_llama3():
    inv = P.rope_inv_freq(TINY_A)
    want = torch.tensor([10000.0 ** (-2 * j / 16) for j in range(8)])
    torch.testing.assert_close(inv, want, atol=0, rtol=1e-6)
    cfg = TINY_B
    s = cfg["rope_scaling"]
    inv = P.rope_inv_freq(cfg)
    hd, orig = cfg["head_dim"], s["original_max_position_embeddings"]
    kinds = set()
    for j in range(hd // 2):
        f = cfg["rope_theta"] ** (-2 * j / hd)
        wavelen = 2 * math.pi / f
        if wavelen > orig / s["low_freq_factor"]:
            want, kind = f / s["factor"], "slowed"
        elif wavelen < orig / s["high_freq_factor"]:
            want, kind = f, "kept"
        else:
            smooth = (orig / wavelen - s["low_freq_factor"]) / (s["high_freq_factor"] - s["low_freq_factor"])
            want, kind = (1 - smooth) * f / s["factor"] + smooth * f, "blended"
        kinds.add(kind)
        assert abs(float(inv[j]) - want) <= 2e-6 * want
    assert kinds == {"slowed", "kept", "blended"}  # the configuration exercises all three bands


def test_rotation_layout_is_half_split():
    x = torch.arange(8.0)[None, None]
    cos, sin = torch.zeros(1, 8), torch.ones(1, 8)
    torch.testing.assert_close(P.apply_rope(x, cos, sin)[0, 0], torch.tensor([-4., -5., -6., -7., 0., 1., 2., 3.]))
    cos, sin = P.rope_angles(torch.tensor([0.5, 0.25]), torch.tensor([0, 3]))
    assert cos.shape == (2, 4) and torch.equal(cos[:, :2], cos[:, 2:])
    torch.testing.assert_close(sin[1], torch.tensor([math.sin(1.5), math.sin(0.75)] * 2))


def test_attention_is_causal_grouped_and_scaled():
    torch.manual_seed(0)
    nh, nkv, t, hd = 6, 2, 9, 8
    q, k, v = torch.randn(nh, t, hd), torch.randn(nkv, t, hd), torch.randn(nkv, t, hd)
    out = P.attention(q, k, v)
    for h in range(nh):
        for i in range(t):
            scores = torch.tensor([float(q[h, i] @ k[h // 3, j]) / math.sqrt(hd) for j in range(i + 1)])
            want = (scores.softmax(0)[:, None] * v[h // 3, : i + 1]).sum(0)
            torch.testing.assert_close(out[h, i], want, atol=1e-5, rtol=1e-5)
    windowed = P.attention(q, k, v, window=3)
    scores = torch.tensor([float(q[0, 8] @ k[0, j]) / math.sqrt(hd) for j in (6, 7, 8)])
    torch.testing.assert_close(windowed[0, 8], (scores.softmax(0)[:, None] * v[0, 6:9]).sum(0), atol=1e-5, rtol=1e-5)


def test_swiglu_formula():
    w = {"m.gate_proj.weight": torch.randn(7, 5), "m.up_proj.weight": torch.randn(7, 5),
         "m.down_proj.weight": torch.randn(5, 7)}
    x = torch.randn(3, 5)
    g, u = x @ w["m.gate_proj.weight"].t(), x @ w["m.up_proj.weight"].t()
    want = (torch.nn.functional.silu(g) * u) @ w["m.down_proj.weight"].t()
    torch.testing.assert_close(P.swiglu(w, "m", x), want, atol=1e-5, rtol=1e-5)


def test_tied_and_untied_heads_and_prefix_property():
    for cfg in (TINY_A, TINY_B):
        weights = helpers.make_weights(cfg, seed=1)
        ids = helpers.random_tokens(cfg, 20, 5)
        full = P.logits_for(cfg, weights, ids)
        assert full.shape == (20, cfg["vocab_size"])
        # causal: the logits of a prefix do not depend on what follows
        torch.testing.assert_close(P.logits_for(cfg, weights, ids[:11]), full[:11], atol=1e-5, rtol=1e-5)
    assert "lm_head.weight" not in helpers.make_weights(TINY_A) and "lm_head.weight" in helpers.make_weights(TINY_B)


def test_greedy_generation_stops_at_a_stop_id():
    weights = helpers.make_weights(TINY_A, seed=2)
    prompt = helpers.random_tokens(TINY_A, 6, 9)
    free = P.greedy_generate(TINY_A, weights, prompt, 6)
    assert len(free) == 6
    stopped = P.greedy_generate(TINY_A, weights, prompt, 6, stop_ids=(free[2],))
    assert stopped == free[: free.index(free[2]) + 1]
