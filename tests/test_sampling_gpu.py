"""The sampling kernel against its plain reference (same uniforms, same order of operations)."""

from __future__ import annotations

import pytest
import torch

from tests.ref_ops import RefOps, philox_uniforms

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from inference_engine_b200.kernels import get_ops

    return get_ops("cuda")


@pytest.mark.parametrize("rows,vocab", [(1, 256), (7, 331), (64, 128256), (3, 50001)])
def test_argmax_lowest_index_on_ties(ops, rows, vocab):
    logits = torch.randn(rows, vocab, device="cuda")
    logits[0, vocab // 3] = 50.0
    logits[0, vocab - 1] = 50.0  # a tie: the lower index wins, as torch.argmax
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    ops.argmax(logits, out)
    assert out.tolist() == logits.argmax(-1).tolist()
    assert out[0].item() == vocab // 3


def _params(rows, device="cuda", **kw):
    f = lambda v: torch.full((rows,), v, dtype=torch.float32, device=device)  # noqa: E731
    out = dict(temperature=f(kw.get("temperature", 0.8)),
               seeds=torch.arange(rows, dtype=torch.int64, device=device) + 7_000_000_000,
               draws=torch.arange(rows, dtype=torch.int64, device=device) * 3)
    if "top_k" in kw:
        out["top_k"] = torch.full((rows,), kw["top_k"], dtype=torch.int32, device=device)
    for name in ("top_p", "min_p"):
        if name in kw:
            out[name] = f(kw[name])
    return out


@pytest.mark.parametrize("vocab", [331, 5000, 128256])
@pytest.mark.parametrize("kw", [dict(), dict(top_k=20), dict(top_p=0.7), dict(min_p=0.05),
                                dict(top_k=50, top_p=0.9, min_p=0.01), dict(temperature=1.7, top_k=3)])
def test_sampling_matches_reference(ops, vocab, kw):
    rows = 6
    g = torch.Generator(device="cuda").manual_seed(vocab)
    logits = torch.randn(rows, vocab, device="cuda", generator=g) * 2.5
    params = _params(rows, **kw)
    got = torch.empty(rows, dtype=torch.int32, device="cuda")
    lp = torch.empty(rows, device="cuda")
    ops.sample(logits, got, logprob=lp, **params)
    want = torch.empty(rows, dtype=torch.int32)
    want_lp = torch.empty(rows)
    RefOps().sample(logits, want, logprob=want_lp, **{k: v.cpu() for k, v in params.items()})
    assert got.tolist() == want.tolist()
    torch.testing.assert_close(lp.cpu(), want_lp, atol=1e-4, rtol=1e-4)


def test_mixed_greedy_and_sampled_rows_with_penalty(ops):
    rows, vocab = 4, 1000
    logits = torch.randn(rows, vocab, device="cuda") * 2
    params = _params(rows)
    params["temperature"][1] = 0.0  # a greedy row among sampled ones
    params["penalty"] = torch.tensor([1.0, 1.5, 2.0, 1.0], device="cuda")
    seen = torch.zeros(rows, (vocab + 31) // 32, dtype=torch.int32, device="cuda")
    best = int(logits[1].argmax())
    seen[1, best // 32] = 1 << (best % 32) if best % 32 < 31 else -(1 << 31)
    seen[2, :] = -1  # every token was seen
    params["seen_bits"] = seen
    got = torch.empty(rows, dtype=torch.int32, device="cuda")
    ops.sample(logits, got, **params)
    want = torch.empty(rows, dtype=torch.int32)
    RefOps().sample(logits, want, **{k: v.cpu() for k, v in params.items()})
    assert got.tolist() == want.tolist()


def test_sampling_follows_the_distribution(ops):
    """Many draws of one row: empirical frequencies match softmax(logits / T) restricted to
    the top-k set (a chi-square style bound)."""
    vocab, n, temp, k = 50, 20000, 0.7, 8
    logits = torch.randn(1, vocab, device="cuda") * 1.5
    rep = logits.expand(n, vocab).contiguous()
    params = dict(temperature=torch.full((n,), temp, device="cuda"),
                  top_k=torch.full((n,), k, dtype=torch.int32, device="cuda"),
                  seeds=torch.full((n,), 42, dtype=torch.int64, device="cuda"),
                  draws=torch.arange(n, dtype=torch.int64, device="cuda"))
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    ops.sample(rep, out, **params)
    z = logits[0] / temp
    kth = z.topk(k).values[-1]
    probs = torch.where(z >= kth, z, torch.tensor(float("-inf"), device="cuda")).softmax(-1)
    freq = torch.bincount(out.long(), minlength=vocab).float() / n
    assert float((freq[probs == 0]).sum()) == 0.0
    assert float((freq - probs).abs().max()) < 4 * (0.25 / n) ** 0.5 + 1e-3


def test_uniforms_are_inside_the_open_interval():
    u = philox_uniforms(123, 5, 100000)
    assert u.min() > 0.0 and u.max() < 1.0
    assert abs(float(u.mean()) - 0.5) < 0.01
