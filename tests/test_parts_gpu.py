"""Each part of a layer alone on the GPU against the plain implementation's function for it:
norm, position encoding, attention mixer over the paged cache, feed-forward, block, embedding
and head -- in 32-bit and bfloat16, at the sizes of tiny B and C."""

from __future__ import annotations

import pytest
import torch

from inference_engine_b200.config.spec import PartSpec
from inference_engine_b200.parts import BuildEnv, CacheBinding, build_part
from tests import helpers as H
from tests import plain_llama as P
from tests.tiny_configs import TINY_B, TINY_C

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def _tol(dtype):
    return dict(atol=3e-5, rtol=1e-4) if dtype == "float32" else dict(atol=4e-2, rtol=4e-2)


def _total(t):
    """A part may hand back its output as partial sums ``[S, N, hidden]`` (the pieces of a
    matrix product that was split along its inner dimension); the next norm adds them."""
    return t.float().sum(0) if t.dim() == 3 else t.float()


class _Ctx:
    """The least a part needs of a step: kernels, buffers and index vectors."""

    def __init__(self, dtype, n):
        from inference_engine_b200.engine.workspace import Workspace
        from inference_engine_b200.kernels import get_ops

        self.ops, self.ws, self.num_tokens = get_ops("cuda"), Workspace("cuda"), n


def _env(cfg, dtype, positions=None):
    return BuildEnv(cfg["hidden_size"], dtype, cfg["max_position_embeddings"], positions or {}, "cuda")


@pytest.mark.parametrize("dtype", DTYPES)
def test_rms_norm_part(dtype):
    env = _env(TINY_C, dtype)
    norm = build_part("norm", PartSpec("rms", {"weight": "w", "eps": 3e-6}), env)
    assert list(norm.weights()) == ["w"] and norm.weights()["w"].shape == (80,)
    w = (1 + 0.1 * torch.randn(80)).bfloat16()
    norm.bind({"w": w.cuda()}, env)
    h, delta = torch.randn(9, 80, device="cuda"), torch.randn(9, 80, device="cuda")
    h0 = h.clone()
    out = norm.add_norm(h, delta, _Ctx(dtype, 9))
    torch.testing.assert_close(h, h0 + delta)
    torch.testing.assert_close(out.float().cpu(), P.rms_norm((h0 + delta).cpu(), w, 3e-6), **_tol(dtype))


def test_rotary_part_tables():
    for cfg in (TINY_B, TINY_C):
        env = _env(cfg, "float32")
        s = cfg.get("rope_scaling")
        scaling = None
        if s:
            scaling = {"factor": s["factor"], "low_freq_factor": s["low_freq_factor"],
                       "high_freq_factor": s["high_freq_factor"],
                       "original_max_position_embeddings": s["original_max_position_embeddings"]}
        rot = build_part("position", PartSpec("rotary", {"rotary_dim": cfg["head_dim"],
                                                          "theta": cfg["rope_theta"], "scaling": scaling}), env)
        rot.bind({}, env)
        table = rot.rotary_table().cpu()
        assert table.shape == (cfg["max_position_embeddings"], 2, cfg["head_dim"] // 2)
        pos = torch.arange(cfg["max_position_embeddings"])
        cos, sin = P.rope_angles(P.rope_inv_freq(cfg), pos)
        half = cfg["head_dim"] // 2
        torch.testing.assert_close(table[:, 0], cos[:, :half], atol=2e-6, rtol=0)
        torch.testing.assert_close(table[:, 1], sin[:, :half], atol=2e-6, rtol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cfg", [TINY_B, TINY_C], ids=["B", "C"])
def test_attention_mixer_over_the_paged_cache(cfg, dtype):
    """The mixer alone: a whole sequence in one step, then the same sequence in two portions
    and a decoded token, against the plain attention block."""
    from inference_engine_b200.cache import CacheManager, CacheStorage, PagedGroupSpec
    from inference_engine_b200.engine.batch import StepEntry
    from inference_engine_b200.engine.runner import ModelRunner

    weights = H.make_weights(cfg, seed=9)
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    s = cfg["rope_scaling"]
    scaling = {k: s[k] for k in ("factor", "low_freq_factor", "high_freq_factor", "original_max_position_embeddings")}
    env = _env(cfg, dtype)
    rot = build_part("position", PartSpec("rotary", {"rotary_dim": hd, "theta": cfg["rope_theta"], "scaling": scaling}), env)
    rot.bind({}, env)
    env.positions = {"rotary": rot}
    p = "model.layers.1.self_attn"
    mixer = build_part("mixer", PartSpec("paged_attention", {
        "q_proj": f"{p}.q_proj.weight", "k_proj": f"{p}.k_proj.weight", "v_proj": f"{p}.v_proj.weight",
        "o_proj": f"{p}.o_proj.weight", "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd,
        "position": "rotary"}), env)
    mixer.bind({n: weights[n].cuda() for n in mixer.weights()}, env)
    req = mixer.cache_request()
    assert (req.num_kv_heads, req.head_dim, req.window) == (nkv, hd, None)

    class OneMixer:  # the smallest "model": the runner only needs groups and a forward
        paged_groups, state_groups = [PagedGroupSpec(1, nkv, hd, None)], []

    t = 45
    x = torch.randn(t, cfg["hidden_size"]) * 0.7
    cos, sin = P.rope_angles(P.rope_inv_freq(cfg), torch.arange(t))
    xq = x.to(env.torch_dtype).float()
    want = P.attention_block(cfg, weights, p, xq, cos, sin)
    cache = CacheManager(OneMixer.paged_groups, [], 16, 8, 2)
    storage = CacheStorage(cache, env.torch_dtype, "cuda")
    from inference_engine_b200.kernels import get_ops

    runner = ModelRunner(OneMixer, cache, storage, get_ops("cuda"), "cuda", 64, 2)
    for portions in ([t], [20, 24, 1]):
        cache.add_request("a")
        outs, pos = [], 0
        for n in portions:
            cache.grow("a", pos, pos + n)
            ctx, _ = runner.build_context([StepEntry("a", [0] * n, pos, [])])
            out = mixer.forward(x[pos:pos + n].cuda().to(env.torch_dtype), ctx, CacheBinding(0, 0))
            outs.append(_total(out).cpu().clone())
            pos += n
        torch.testing.assert_close(torch.cat(outs), want, **_tol(dtype))
        cache.free("a")
    get_ops("cuda").check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_part(dtype):
    cfg = TINY_C
    weights = H.make_weights(cfg, seed=10)
    env = _env(cfg, dtype)
    p = "model.layers.0.mlp"
    ffn = build_part("feed_forward", PartSpec("swiglu", {
        "gate_proj": f"{p}.gate_proj.weight", "up_proj": f"{p}.up_proj.weight",
        "down_proj": f"{p}.down_proj.weight", "intermediate_size": cfg["intermediate_size"]}), env)
    ffn.bind({n: weights[n].cuda() for n in ffn.weights()}, env)
    x = (torch.randn(13, cfg["hidden_size"]) * 2).to(env.torch_dtype)
    out = ffn.forward(x.cuda(), _Ctx(dtype, 13))
    torch.testing.assert_close(_total(out).cpu(), P.swiglu(weights, p, x.float()), **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_tied_head(dtype):
    cfg = TINY_C
    env = _env(cfg, dtype)
    table = (torch.randn(cfg["vocab_size"], cfg["hidden_size"]) * 0.5).bfloat16()
    emb = build_part("embedding", PartSpec("token", {"weight": "e", "vocab_size": cfg["vocab_size"]}), env)
    emb.bind({"e": table.cuda()}, env)
    ids = torch.tensor([5, 330, 0, 77], dtype=torch.int32, device="cuda")
    h = emb.forward(ids, _Ctx(dtype, 4))
    assert h.dtype == torch.float32 and torch.equal(h.cpu(), table.float()[ids.cpu().long()])
    head = build_part("head", PartSpec("linear", {"weight": None, "vocab_size": cfg["vocab_size"]}), env)
    assert head.weights() == {}
    head.tie(emb.table)
    x = torch.randn(4, cfg["hidden_size"]).to(env.torch_dtype)
    logits = head.forward(x.cuda(), _Ctx(dtype, 4))
    assert logits.dtype == torch.float32
    torch.testing.assert_close(logits.cpu(), x.float() @ table.float().t(), **_tol(dtype))
