"""Each CUDA kernel alone against its plain PyTorch reference (tests/ref_ops.py), at sizes
other than the engine's test models: widths and vocabularies that are no power of two, odd
head counts and groups, head sizes in steps of 16."""

from __future__ import annotations

import types

import pytest
import torch

from tests.ref_ops import RefOps

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from inference_engine_b200.kernels import get_ops

    return get_ops("cuda")


def _tol(dtype):
    return dict(atol=2e-6, rtol=2e-6) if dtype == torch.float32 else dict(atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab,hidden,n", [(331, 80, 7), (1000, 2048, 33), (50, 24, 1)])
def test_embedding(ops, dtype, vocab, hidden, n):
    table = torch.randn(vocab, hidden, device="cuda").to(dtype)
    ids = torch.randint(0, vocab, (n,), device="cuda", dtype=torch.int32)
    got = torch.empty(n, hidden, device="cuda")
    want = torch.empty_like(got)
    ops.embedding(table, ids, got)
    RefOps().embedding(table, ids, want)
    assert torch.equal(got, want)
    ops.check_errors()


def test_embedding_reports_a_bad_token_id(ops):
    from inference_engine_b200.kernels import KernelError

    table = torch.randn(10, 16, device="cuda")
    ids = torch.tensor([3, 10], device="cuda", dtype=torch.int32)
    out = torch.empty(2, 16, device="cuda")
    ops.embedding(table, ids, out)
    with pytest.raises(KernelError, match="token id"):
        ops.check_errors()
    ops.check_errors()  # the error word was cleared


@pytest.mark.parametrize("out_dtype", DTYPES)
@pytest.mark.parametrize("n,hidden,eps", [(5, 80, 3e-6), (33, 2048, 1e-5), (1, 96, 1e-6), (3, 4100, 1e-5)])
def test_rmsnorm_with_residual_add(ops, out_dtype, n, hidden, eps):
    h = torch.randn(n, hidden, device="cuda") * 3
    delta = torch.randn(n, hidden, device="cuda")
    w = 1 + 0.1 * torch.randn(hidden, device="cuda")
    for use_delta in (True, False):
        h1, h2 = h.clone(), h.clone()
        got = torch.empty(n, hidden, device="cuda", dtype=out_dtype)
        want = torch.empty_like(got)
        ops.rmsnorm(h1, delta if use_delta else None, w, eps, got)
        RefOps().rmsnorm(h2, delta if use_delta else None, w, eps, want)
        assert torch.equal(h1, h2)  # the residual stream itself: one add, exact
        torch.testing.assert_close(got.float(), want.float(), **_tol(out_dtype))
    rows = torch.tensor([n - 1, 0, n // 2], device="cuda", dtype=torch.int32)
    h1 = h.clone()
    got = torch.empty(3, hidden, device="cuda", dtype=out_dtype)
    want = torch.empty_like(got)
    ops.rmsnorm(h1, delta, w, eps, got, rows)
    RefOps().rmsnorm(h.clone(), delta, w, eps, want, rows)
    assert torch.equal(h1, h)  # selected rows: nothing is written back
    torch.testing.assert_close(got.float(), want.float(), **_tol(out_dtype))


@pytest.mark.parametrize("out_dtype", DTYPES)
@pytest.mark.parametrize("hidden", [80, 2048, 4100])
def test_consumers_add_the_parts_of_a_split_matrix_product(ops, out_dtype, hidden):
    """Norm, rotary/cache write and activation accept their input as S partial sums."""
    n, parts = 5, 3
    h = torch.randn(n, hidden, device="cuda")
    delta = torch.randn(parts, n, hidden, device="cuda")
    w = torch.randn(hidden, device="cuda")
    h1, h2 = h.clone(), h.clone()
    got = torch.empty(n, hidden, device="cuda", dtype=out_dtype)
    want = torch.empty_like(got)
    ops.rmsnorm(h1, delta, w, 1e-5, got)
    RefOps().rmsnorm(h2, delta, w, 1e-5, want)
    torch.testing.assert_close(h1, h2, atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(got.float(), want.float(), **_tol(out_dtype))
    inter = hidden // 2 if hidden % 2 == 0 else hidden
    gu = torch.randn(parts, n, 2 * inter, device="cuda")
    got = torch.empty(n, inter, device="cuda", dtype=out_dtype)
    want = torch.empty_like(got)
    ops.silu_mul(gu, got)
    RefOps().silu_mul(gu, want)
    torch.testing.assert_close(got.float(), want.float(), **_tol(out_dtype))
    nh, nkv, hd, ps = 4, 2, 16, 8
    qkv = torch.randn(parts, n, (nh + 2 * nkv) * hd, device="cuda")
    positions = torch.arange(n, device="cuda", dtype=torch.int32)
    ang = torch.rand(16, hd // 2, device="cuda")
    table = torch.stack((ang.cos(), ang.sin()), dim=1).contiguous()
    slots = torch.arange(n, device="cuda", dtype=torch.int32) + 3
    # rotary over the whole head (the vector kernel) and over its first 8 dims only (the general one)
    for rotary_dim, tab in ((hd, table), (8, table[:, :, :4].contiguous())):
        res = []
        for impl in (ops, RefOps()):
            q = torch.zeros(n, nh * hd, device="cuda", dtype=out_dtype)
            k = torch.zeros(2, nkv, ps, hd, device="cuda", dtype=out_dtype)
            v = torch.zeros_like(k)
            impl.rope_kv_write(qkv, positions, tab, rotary_dim, q, k, v, slots, nh, nkv, hd, ps)
            res.append((q, k, v))
        for a, b in zip(*res):
            torch.testing.assert_close(a.float(), b.float(), **_tol(out_dtype))


def test_rmsnorm_row_does_not_depend_on_the_batch(ops):
    h = torch.randn(64, 2048, device="cuda")
    w = torch.randn(2048, device="cuda")
    full = torch.empty(64, 2048, device="cuda")
    ops.rmsnorm(h.clone(), None, w, 1e-5, full)
    one = torch.empty(1, 2048, device="cuda")
    ops.rmsnorm(h[17:18].clone(), None, w, 1e-5, one)
    assert torch.equal(full[17:18], one)


@pytest.mark.parametrize("m,n,k", [(1, 331, 80), (7, 192, 64), (70, 512, 96), (33, 1000, 1030), (130, 65, 17)])
def test_gemm_f32(ops, m, n, k):
    x = torch.randn(m, k, device="cuda")
    w = torch.randn(n, k, device="cuda")
    got = torch.empty(m, n, device="cuda")
    ops.linear(x, w, got)
    want = (x.double() @ w.double().t()).float()
    torch.testing.assert_close(got, want, atol=1e-4 * k ** 0.5, rtol=1e-5)
    one = torch.empty(1, n, device="cuda")
    ops.linear(x[m // 2: m // 2 + 1].contiguous(), w, one)
    assert torch.equal(one, got[m // 2: m // 2 + 1])  # a row's result does not depend on M


@pytest.mark.parametrize("out_dtype", DTYPES)
@pytest.mark.parametrize("m,n,k", [(1, 328, 80), (7, 192, 64), (70, 512, 96), (33, 1000, 1032)])
def test_linear_bf16(ops, out_dtype, m, n, k):
    x = torch.randn(m, k, device="cuda").bfloat16()
    w = torch.randn(n, k, device="cuda").bfloat16()
    got = torch.empty(m, n, device="cuda", dtype=out_dtype)
    ops.linear(x, w, got)
    want = x.double() @ w.double().t()
    tol = dict(atol=1e-3 * k ** 0.5, rtol=1e-5) if out_dtype == torch.float32 else dict(atol=0.02 * k ** 0.5, rtol=1e-2)
    torch.testing.assert_close(got.double(), want, **tol)


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("n,k", [(3072, 2048), (2048, 8192), (331, 80), (192, 64), (512, 96), (1000, 1032), (16384, 2048)])
def test_tma_fed_gemm_for_few_rows(ops, m, n, k, monkeypatch):
    """The TMA-fed weight-streaming product: any N (tiles of 128 with a ragged edge), any K
    that is a multiple of 8 (blocks of 64 with a ragged edge), with and without k splits."""
    from inference_engine_b200.engine.workspace import Workspace

    monkeypatch.setattr(ops, "blas_split_k", False)  # (9 to 16 rows with a long inner dimension would go to the library)

    x = torch.randn(m, k, device="cuda").bfloat16()
    w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
    want = x.double() @ w.double().t()
    ws = Workspace("cuda")
    saved, ops.few_row_gemm = ops.few_row_gemm, "tma"
    try:
        split = ops.linear(x, w, ws=ws, tag="t", out_dtype=torch.float32, allow_split=True)
        per, splits = ops.tma_split(n, k)
        assert split.shape == ((splits, m, n) if splits > 1 else (m, n))
        total = split.sum(0) if split.dim() == 3 else split
        torch.testing.assert_close(total.double(), want, atol=2e-4 * k ** 0.5, rtol=1e-5)
        for out_dtype in DTYPES:
            out = torch.empty(m, n, device="cuda", dtype=out_dtype)
            assert ops.linear(x, w, out) is out
            tol = dict(atol=2e-4 * k ** 0.5, rtol=1e-5) if out_dtype == torch.float32 else dict(atol=0.01 * k ** 0.5, rtol=1e-2)
            torch.testing.assert_close(out.double(), want, **tol)
        ops.check_errors()
    finally:
        ops.few_row_gemm = saved


@pytest.mark.parametrize("m", [17, 33, 64, 100, 128, 200, 256])
@pytest.mark.parametrize("n,k", [(3072, 2048), (2048, 8192), (328, 128), (192, 64), (1000, 1024), (16384, 2048)])
def test_tcgen05_gemm_for_a_batch_of_decode_tokens(ops, m, n, k, monkeypatch):
    """17 to 256 rows: features are the rows of tcgen05.mma, tokens its columns; any N (tiles of
    128 with a ragged edge), K a multiple of 64, with and without k splits, 32-bit and bfloat16
    results; twice, so that tensor memory must have been given back."""
    from inference_engine_b200.engine.workspace import Workspace

    monkeypatch.setattr(ops, "blas_split_k", False)  # (the routing's first choice for these shapes: tested below)
    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    x = torch.randn(m, k, device="cuda", generator=g).bfloat16()
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.05).bfloat16()
    want = x.double() @ w.double().t()
    ws = Workspace("cuda")
    saved = ops.batch_gemm, ops.batch_gemm_rows, ops.batch_gemm_max_tiles, ops.batch_gemm_min_k, ops.batch_gemm_one_round
    ops.batch_gemm, ops.batch_gemm_rows, ops.batch_gemm_max_tiles, ops.batch_gemm_min_k = True, 256, 1 << 20, 0
    ops.batch_gemm_one_round = False
    launches = ops.launches
    try:
        for _ in range(2):
            split = ops.linear(x, w, ws=ws, tag="t", out_dtype=torch.float32, allow_split=True)
            per, splits = ops.tma_split(n, k)
            assert split.shape == ((splits, m, n) if splits > 1 else (m, n))
            total = split.sum(0) if split.dim() == 3 else split
            torch.testing.assert_close(total.double(), want, atol=2e-4 * k ** 0.5, rtol=1e-5)
            for out_dtype in DTYPES:
                out = torch.empty(m, n, device="cuda", dtype=out_dtype)
                assert ops.linear(x, w, out) is out
                tol = dict(atol=2e-4 * k ** 0.5, rtol=1e-5) if out_dtype == torch.float32 else dict(atol=0.01 * k ** 0.5, rtol=1e-2)
                torch.testing.assert_close(out.double(), want, **tol)
        assert ops.launches - launches == 6  # every product ran this kernel, none the vendor library
        ops.check_errors()
    finally:
        (ops.batch_gemm, ops.batch_gemm_rows, ops.batch_gemm_max_tiles, ops.batch_gemm_min_k,
         ops.batch_gemm_one_round) = saved


@pytest.mark.parametrize("m", [9, 16, 17, 64, 130, 256, 512, 1024])
@pytest.mark.parametrize("n,k", [(2048, 8192), (2048, 2048), (3072, 2048), (4096, 4096), (1000, 1536), (16384, 2048)])
def test_narrow_products_are_cut_along_k_for_the_library(ops, m, n, k):
    """Products of more than 8 rows with few output features go to the library as one batched
    product over slices of the inner dimension (`CudaOps.blas_split`); the consumer adds the parts.
    The parts sum to the product; shapes that are not cut come back whole."""
    from inference_engine_b200.engine.workspace import Workspace

    g = torch.Generator(device="cuda").manual_seed(m * 7 + n + k)
    x = torch.randn(m, k, device="cuda", generator=g).bfloat16()
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.05).bfloat16()
    want = x.double() @ w.double().t()
    ws = Workspace("cuda")
    parts = ops.blas_split(m, n, k)
    assert parts in (1, 2, 4, 8) and (parts == 1 or (k // parts >= 256 and k % parts == 0))
    assert ops.blas_split(32, 2048, 8192) == 8 and ops.blas_split(64, 2048, 8192) == 4 and ops.blas_split(256, 2048, 8192) == 4
    assert ops.blas_split(512, 2048, 8192) == 2 and ops.blas_split(513, 2048, 8192) == 1
    assert ops.blas_split(64, 16384, 2048) == 1 and ops.blas_split(2048, 2048, 8192) == 1
    got = ops.linear(x, w, ws=ws, tag="t", out_dtype=torch.float32, allow_split=True)
    if parts > 1 and not (m <= 16 and k < 4096):
        assert got.shape == (parts, m, n)
    total = got.sum(0) if got.dim() == 3 else got
    torch.testing.assert_close(total.double(), want, atol=2e-4 * k ** 0.5, rtol=1e-5)
    # the consumers add the parts in order: a norm over them gives the norm of the sum
    if got.dim() == 3 and n % 8 == 0:
        h = torch.randn(m, n, device="cuda", generator=g)
        weight = torch.ones(n, device="cuda")
        out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        h_got = h.clone()
        ops.rmsnorm(h_got, got, weight, 1e-5, out)
        x_sum = h.double() + want
        want_norm = x_sum * torch.rsqrt(x_sum.pow(2).mean(-1, keepdim=True) + 1e-5)
        torch.testing.assert_close(out.double(), want_norm, atol=2e-2, rtol=2e-2)
    ops.check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,rd,ps", [(4, 2, 16, 16, 16), (3, 1, 32, 32, 8), (5, 5, 48, 48, 4),
                                             (32, 8, 64, 64, 16), (6, 2, 80, 32, 16), (2, 1, 128, 0, 32)])
def test_rope_and_cache_write(ops, dtype, nh, nkv, hd, rd, ps):
    n, maxpos = 37, 500
    pages = -(-n // ps) + 3
    qkv = torch.randn(n, (nh + 2 * nkv) * hd, device="cuda")
    positions = torch.randint(0, maxpos, (n,), device="cuda", dtype=torch.int32)
    table = None
    if rd:
        ang = torch.rand(maxpos, rd // 2, device="cuda") * 6.28
        table = torch.stack((ang.cos(), ang.sin()), dim=1).contiguous()
    slots = torch.randperm(pages * ps, device="cuda")[:n].to(torch.int32)
    res = []
    for impl in (ops, RefOps()):
        q = torch.zeros(n, nh * hd, device="cuda", dtype=dtype)
        k = torch.zeros(pages, nkv, ps, hd, device="cuda", dtype=dtype)
        v = torch.zeros_like(k)
        impl.rope_kv_write(qkv, positions, table, rd, q, k, v, slots, nh, nkv, hd, ps)
        res.append((q, k, v))
    for a, b in zip(*res):
        torch.testing.assert_close(a.float(), b.float(), **_tol(dtype))
    # a run that borrows another layer's cache rotates queries and writes nothing
    q = torch.zeros(n, nh * hd, device="cuda", dtype=dtype)
    k = torch.zeros(pages, nkv, ps, hd, device="cuda", dtype=dtype)
    v = torch.zeros_like(k)
    ops.rope_kv_write(qkv, positions, table, rd, q, k, v, None, nh, nkv, hd, ps)
    torch.testing.assert_close(q.float(), res[1][0].float(), **_tol(dtype))
    assert not k.any() and not v.any()
    ops.check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,inter", [(5, 192), (33, 8192), (1, 321), (64, 1000)])
def test_silu_mul(ops, dtype, n, inter):
    gu = (torch.randn(n, 2 * inter, device="cuda") * 3).to(dtype)
    got = torch.empty(n, inter, device="cuda", dtype=dtype)
    want = torch.empty_like(got)
    ops.silu_mul(gu, got)
    RefOps().silu_mul(gu, want)
    torch.testing.assert_close(got.float(), want.float(), **_tol(dtype))
    # gates and ups alternating in blocks of 8 or 16 values: the same numbers from other places
    plain = want.clone()
    for block in (8, 16):
        if inter % block:
            continue
        mixed = torch.stack([gu[:, :inter].view(n, inter // block, block), gu[:, inter:].view(n, inter // block, block)],
                            dim=2).reshape(n, 2 * inter).contiguous()
        ops.silu_mul(mixed, got, block)
        RefOps().silu_mul(mixed, want, block)
        torch.testing.assert_close(got.float(), want.float(), **_tol(dtype))
        assert torch.equal(want, plain)


@pytest.mark.parametrize("m", [1, 5, 8, 9, 16])
@pytest.mark.parametrize("inter,k", [(8192, 2048), (176, 96), (320, 64), (1008, 1032), (11008, 2048)])
def test_gated_product_applies_the_activation_in_the_kernel(ops, m, inter, k):
    """A few rows through the gated feed-forward's first half: the TMA-fed kernel on a matrix whose
    gate and up rows alternate in blocks of 16 gives silu(x gate^T) * (x up^T), also where the
    last tile of 128 rows is not full; other layouts and sizes take the two-kernel way."""
    from inference_engine_b200.engine.workspace import Workspace

    g = torch.Generator(device="cuda").manual_seed(inter + k + m)
    x = torch.randn(m, k, device="cuda", generator=g).bfloat16()
    gate = (torch.randn(inter, k, device="cuda", generator=g) * 0.05).bfloat16()
    up = (torch.randn(inter, k, device="cuda", generator=g) * 0.05).bfloat16()
    a, b = x.double() @ gate.double().t(), x.double() @ up.double().t()
    want = a / (1 + torch.exp(-a)) * b
    ws = Workspace("cuda")
    block = ops.GATE_BLOCK
    stacked = torch.stack([gate.view(inter // block, block, k), up.view(inter // block, block, k)], dim=1)
    stacked = stacked.reshape(2 * inter, k).contiguous()
    before = ops.launch_counts.get("gemm_tma_gated", 0)
    got = ops.gated_linear(x, stacked, block, ws=ws, tag="t", out_dtype=torch.bfloat16)
    fused = ops.launch_counts.get("gemm_tma_gated", 0) - before
    assert fused == (1 if (m <= 8 or -(-2 * inter // 128) <= ops.tma_max_tiles_wide) else 0)
    torch.testing.assert_close(got.double(), want, atol=0.01 * k ** 0.5 * 0.05 * 3, rtol=2e-2)
    halves = ops.gated_linear(x, torch.cat([gate, up]).contiguous(), 0, ws=ws, tag="u", out_dtype=torch.bfloat16)
    assert ops.launch_counts.get("gemm_tma_gated", 0) - before == fused  # the plain layout: two kernels
    torch.testing.assert_close(halves.double(), want, atol=0.01 * k ** 0.5 * 0.05 * 3, rtol=2e-2)
    ops.check_errors()


def _attention_case(nh, nkv, hd, ps, q_lens, ctx_lens, dtype, seed=0, spike=None):
    """A random paged cache with shuffled pages and a step of len(q_lens) sequences."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    b = len(q_lens)
    pages_per_seq = [-(-c // ps) for c in ctx_lens]
    total = sum(pages_per_seq) + 3
    perm = torch.randperm(total, device="cuda", generator=g).tolist()
    width = max(pages_per_seq)
    tables = torch.full((b, width), -1, dtype=torch.int32)
    cursor = 0
    for i, n in enumerate(pages_per_seq):
        tables[i, :n] = torch.tensor(perm[cursor:cursor + n], dtype=torch.int32)
        cursor += n
    k = torch.randn(total, nkv, ps, hd, device="cuda", generator=g)
    v = torch.randn(total, nkv, ps, hd, device="cuda", generator=g)
    n_tok = sum(q_lens)
    q = torch.randn(n_tok, nh * hd, device="cuda", generator=g)
    positions, seqs = [], []
    for i, (ql, cl) in enumerate(zip(q_lens, ctx_lens)):
        positions += list(range(cl - ql, cl))
        seqs += [i] * ql
    if spike is not None:
        # One far key per sequence gets a score that stands out for every query of that
        # sequence: the output must be (nearly) that key's value, wherever its page lies.
        for i, key_pos in enumerate(spike):
            page, off = int(tables[i, key_pos // ps]), key_pos % ps
            rows = [t for t in range(n_tok) if seqs[t] == i]
            direction = torch.randn(hd, device="cuda", generator=g)
            direction = direction / direction.norm()
            k[page, :, off] = direction * 40.0
            q.view(n_tok, nh, hd)[rows] = direction * (hd ** 0.5)
    ctx = types.SimpleNamespace(
        num_tokens=n_tok, num_seqs=b,
        positions=torch.tensor(positions, dtype=torch.int32, device="cuda"),
        seq_of_token=torch.tensor(seqs, dtype=torch.int32, device="cuda"),
        cu_q=torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device="cuda"),
        ctx_lens=torch.tensor(ctx_lens, dtype=torch.int32, device="cuda"),
        q_lens=list(q_lens), start_positions=[c - q for c, q in zip(ctx_lens, q_lens)],
        q_starts=[0] + list(torch.tensor(q_lens).cumsum(0))[:-1],
        max_q_len=max(q_lens), max_ctx_len=max(ctx_lens), padded=False)
    return q.to(dtype), k.to(dtype), v.to(dtype), tables.cuda(), ctx


ATTN_SHAPES = [(4, 2, 16, 16), (3, 1, 32, 8), (5, 5, 48, 4), (32, 8, 64, 16), (8, 2, 128, 16),
               (6, 3, 80, 16), (14, 2, 64, 32), (2, 1, 256, 16)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,ps", ATTN_SHAPES)
@pytest.mark.parametrize("window", [0, 37])
def test_paged_attention_mixed_step(ops, dtype, nh, nkv, hd, ps, window):
    q_lens, ctx_lens = [1, 17, 2, 1, 40, 130, 3, 70], [200, 17, 65, 1, 333, 500, 64, 70]
    q, k, v, tables, ctx = _attention_case(nh, nkv, hd, ps, q_lens, ctx_lens, dtype)
    got = torch.empty_like(q)
    want = torch.empty_like(q)
    scale = hd ** -0.5
    ops.paged_attention(q, k, v, tables, ctx, nh, nkv, hd, ps, scale, window, got)
    RefOps().paged_attention(q, k, v, tables, ctx, nh, nkv, hd, ps, scale, window, want)
    tol = dict(atol=2e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(got.float(), want.float(), **tol)
    ops.check_errors()


@pytest.mark.parametrize("nh,nkv,hd,ps", ATTN_SHAPES)
@pytest.mark.parametrize("window", [0, 100])
def test_paged_attention_decode_only_and_prefill_only(ops, nh, nkv, hd, ps, window):
    """bfloat16: a decode-only step (every context length around tile and page edges, cut
    into several splits) and a prefill-only step (portions longer than a 64-token tile, from
    the start of a sequence and from its middle)."""
    dtype = torch.bfloat16
    cases = [([1] * 9, [1, 15, 16, 17, 63, 64, 65, 1000, 257]),
             ([200, 65, 130, 64], [200, 65, 700, 128])]
    for q_lens, ctx_lens in cases:
        q, k, v, tables, ctx = _attention_case(nh, nkv, hd, ps, q_lens, ctx_lens, dtype, seed=3)
        got = torch.empty_like(q)
        want = torch.empty_like(q)
        ops.paged_attention(q, k, v, tables, ctx, nh, nkv, hd, ps, hd ** -0.5, window, got)
        RefOps().paged_attention(q, k, v, tables, ctx, nh, nkv, hd, ps, hd ** -0.5, window, want)
        torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
        general = torch.empty_like(q)
        ops.paged_attention_general(q, k, v, tables, ctx, nh, nkv, hd, ps, hd ** -0.5, window, general)
        torch.testing.assert_close(general.float(), want.float(), atol=2e-2, rtol=2e-2)
    ops.check_errors()


def test_decode_attention_with_many_splits_is_the_same_as_one(ops):
    """A single request fills the GPU: its context is spread over many blocks; the merged
    result equals the unsplit one up to rounding."""
    nh, nkv, hd, ps = 8, 2, 64, 16
    q, k, v, tables, ctx = _attention_case(nh, nkv, hd, ps, [1], [3000], torch.bfloat16, seed=4)
    assert ops.decode_splits(1, nkv, tables.shape[1] * ps) >= 8
    got = torch.empty_like(q)
    ops.paged_attention(q, k, v, tables, ctx, nh, nkv, hd, ps, hd ** -0.5, 0, got)
    want = torch.empty_like(q)
    RefOps().paged_attention(q, k, v, tables, ctx, nh, nkv, hd, ps, hd ** -0.5, 0, want)
    torch.testing.assert_close(got.float(), want.float(), atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("nh,nkv,hd,ps", [(4, 2, 64, 16), (2, 1, 128, 16)])
@pytest.mark.parametrize("far", [True, False])
def test_prefill_attention_over_a_long_context(ops, nh, nkv, hd, ps, far):
    """Prompt portions at the end of contexts of 40,000 and 20,500 tokens (2,500 block-table entries:
    a late query tile needs them all).  One key per request stands out, near the context's start or
    24,000 tokens in: the output must be that key's value, whichever page it lies in."""
    ctx_lens, q_lens = [40000, 20500], [300, 140]
    spike = [77, 1031] if far else [24000, 20400]
    q, k, v, tables, ctx = _attention_case(nh, nkv, hd, ps, q_lens, ctx_lens, torch.bfloat16, seed=21, spike=spike)
    got = torch.empty_like(q)
    before = ops.launch_counts.get("attention_prefill_tc5", 0)
    ops.paged_attention(q, k, v, tables, ctx, nh, nkv, hd, ps, hd ** -0.5, 0, got)
    assert ops.launch_counts.get("attention_prefill_tc5", 0) == before + 1  # (the tcgen05 kernel, not the fallback)
    want = torch.empty_like(q)
    RefOps().paged_attention(q, k, v, tables, ctx, nh, nkv, hd, ps, hd ** -0.5, 0, want)
    torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
    # (the output is that key's value)
    for i, (key_pos, last) in enumerate(zip(spike, (q_lens[0] - 1, sum(q_lens) - 1))):  # (a request's last token sees every key)
        page, off = int(tables[i, key_pos // ps]), key_pos % ps
        value = v[page, :, off].float().repeat_interleave(nh // nkv, dim=0).reshape(-1)
        torch.testing.assert_close(got[last].float(), value, atol=3e-2, rtol=3e-2)
    ops.check_errors()


@pytest.mark.parametrize("nh,nkv,hd,ps", [(32, 8, 64, 16), (8, 2, 128, 16), (5, 5, 48, 4)])
def test_decode_attention_starts_the_requests_blocks_in_a_given_order(ops, nh, nkv, hd, ps, monkeypatch):
    """The by-request decode attention takes the order in which the requests' blocks start (the
    runner gives the longest first): whatever the order, every request gets its own result, bit for
    bit the same (50 requests of one key to thousands: more blocks than the device runs at once)."""
    monkeypatch.setattr(ops, "decode_balanced", "0")
    g = torch.Generator().manual_seed(7)
    ctx_lens = torch.randint(1, 3000, (50,), generator=g).tolist()
    q, k, v, tables, ctx = _attention_case(nh, nkv, hd, ps, [1] * 50, ctx_lens, torch.bfloat16, seed=9)
    want = torch.empty_like(q)
    RefOps().paged_attention(q, k, v, tables, ctx, nh, nkv, hd, ps, hd ** -0.5, 0, want)
    outs = []
    for order in (None, torch.argsort(ctx.ctx_lens, descending=True), torch.randperm(50, generator=g).cuda()):
        ctx.decode_order = None if order is None else order.to(torch.int32)
        got = torch.zeros_like(q)
        ops.paged_attention(q, k, v, tables, ctx, nh, nkv, hd, ps, hd ** -0.5, 0, got)
        torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
        outs.append(got)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    ops.check_errors()


@pytest.mark.parametrize("nh,nkv,hd,ps,window", [(32, 8, 64, 16, 0), (16, 8, 128, 16, 0), (12, 6, 80, 8, 200), (8, 8, 32, 4, 0)])
def test_decode_attention_in_small_blocks(ops, nh, nkv, hd, ps, window):
    """Many requests of about one length, dealt by request to blocks of two or three warps (the launch hints 2, 3):
    the same result as in the larger blocks, against the plain formula; one far key per request
    stands out.  Requests of two tokens and a request the prefill kernel takes are among them."""
    n = 300 // nkv + 3  # (more blocks than two per SM)
    g = torch.Generator().manual_seed(3)
    ctx_lens = torch.randint(500, 600, (n,), generator=g).tolist()
    group = nh // nkv
    q_lens = [1] * n
    q_lens[5], q_lens[n // 2] = (2 if 2 * group <= 16 else 1), 40
    spike = [(c - ql) // 3 for c, ql in zip(ctx_lens, q_lens)]
    q, k, v, tables, ctx = _attention_case(nh, nkv, hd, ps, q_lens, ctx_lens, torch.bfloat16, seed=13, spike=spike)
    want = torch.empty_like(q)
    RefOps().paged_attention(q, k, v, tables, ctx, nh, nkv, hd, ps, hd ** -0.5, window, want)
    outs = []
    for hint in (ops.BY_REQUEST, ops.SMALL_2, ops.SMALL_3):
        got = torch.zeros_like(q)
        ops.paged_attention(q, k, v, tables, ctx, nh, nkv, hd, ps, hd ** -0.5, window, got, ragged=hint)
        torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
        outs.append(got)
    small = [i for i, ql in enumerate(q_lens) if ql * group <= 16]
    rows = torch.cat([torch.arange(int(ctx.cu_q[i]), int(ctx.cu_q[i + 1])) for i in small]).cuda()
    assert max((outs[0][rows] - o[rows]).abs().max() for o in outs[1:]) < 2e-2  # (other warps, another order of the tiles' sums)
    ops.check_errors()


@pytest.mark.parametrize("nh,nkv,hd,ps", [(32, 8, 64, 16), (8, 2, 128, 16), (6, 3, 80, 8), (4, 4, 32, 4)])
@pytest.mark.parametrize("window", [0, 300])
@pytest.mark.parametrize("blocks_per_pair", [1, 2, 3, 32])
def test_decode_attention_deals_ragged_contexts_evenly(ops, nh, nkv, hd, ps, window, blocks_per_pair, monkeypatch):
    """The decode kernel that deals key tiles by length: contexts from one key to thousands in
    one step, portions of one to four tokens, a request in the middle that the prefill kernel
    takes.  However many blocks the tiles are dealt to (as many as there are requests and heads;
    twice or three times as many; all the device runs), every request gets its own result.  One
    far key per request stands out, so a block that took the wrong tiles, or a partial result
    merged into the wrong request, shows."""
    ctx_lens = [1, 5000, 31, 32, 33, 700, 64, 2, 1500, 96, 4097, 12, 257, 640, 9, 3000]
    q_lens = [1, 1, 2, 1, 1, 1, 64, 1, 1, 3, 1, 1, 1, 1, 4, 1]
    group = nh // nkv
    q_lens = [ql if ql == 64 or ql * group <= 16 else 1 for ql in q_lens]
    # a key every query of the portion sees: far back, or in the middle of the window
    spike = [max(0, c - ql - window // 2) if window else (c - ql) // 3 for c, ql in zip(ctx_lens, q_lens)]
    monkeypatch.setattr(ops, "decode_balanced", "1")
    monkeypatch.setattr(ops, "decode_balanced_blocks_per_pair", blocks_per_pair)
    q, k, v, tables, ctx = _attention_case(nh, nkv, hd, ps, q_lens, ctx_lens, torch.bfloat16, seed=11, spike=spike)
    got = torch.empty_like(q)
    want = torch.empty_like(q)
    ops.paged_attention(q, k, v, tables, ctx, nh, nkv, hd, ps, hd ** -0.5, window, got)
    RefOps().paged_attention(q, k, v, tables, ctx, nh, nkv, hd, ps, hd ** -0.5, window, want)
    torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
    ops.check_errors()
    # the launch left its ticket counters at zero: a second one on the same data gives the same
    again = torch.empty_like(q)
    ops.paged_attention(q, k, v, tables, ctx, nh, nkv, hd, ps, hd ** -0.5, window, again)
    assert torch.equal(again, got)


@pytest.mark.parametrize("nh,nkv,hd,ps,seqs,parts", [
    (32, 8, 64, 16, 8, 2), (8, 2, 128, 16, 30, 2), (6, 3, 32, 8, 17, 2), (16, 8, 64, 16, 7, 2),
    (32, 8, 64, 16, 4, 4), (32, 8, 64, 16, 1, 8), (8, 2, 128, 16, 9, 4), (8, 2, 128, 16, 2, 8), (5, 5, 48, 4, 3, 8)])
@pytest.mark.parametrize("window", [0, 300])
def test_splits_of_a_context_merge_through_shared_memory(ops, nh, nkv, hd, ps, seqs, parts, window):
    """Batches for which the decode attention cuts every context in 2, 4 or 8 run the blocks of a
    (request, head) pair as a thread-block cluster that merges through the first block's shared
    memory (head size 128 with 8 parts has no room for that and merges through memory).  The
    result is that of the merge through memory (same sums in the same order: equal bit for bit)
    and the plain attention's; a far key per request stands out; contexts from one key (the later
    blocks have nothing) to thousands, portions of one to four tokens."""
    ctx_lens = ([1, 17, 1024, 333, 2048, 64, 700, 31, 3000, 2, 96, 1500] * 3)[:seqs]
    assert ops.decode_splits(seqs, nkv, -(-max(ctx_lens) // ps) * ps) == parts
    group = nh // nkv
    q_lens = [(1 + i % 4) if (1 + i % 4) * group <= 16 else 1 for i in range(seqs)]
    q_lens = [min(ql, c) for ql, c in zip(q_lens, ctx_lens)]
    spike = [max(0, c - ql - window // 2) if window else (c - ql) // 3 for c, ql in zip(ctx_lens, q_lens)]
    q, k, v, tables, ctx = _attention_case(nh, nkv, hd, ps, q_lens, ctx_lens, torch.bfloat16, seed=5, spike=spike)
    want = torch.empty_like(q)
    RefOps().paged_attention(q, k, v, tables, ctx, nh, nkv, hd, ps, hd ** -0.5, window, want)
    lib = ops._attention_lib(hd)
    outs = []
    try:
        for pair in (8, 0, 8):
            lib.ie_set_decode_pair(pair)
            got = torch.zeros_like(q)
            ops.paged_attention(q, k, v, tables, ctx, nh, nkv, hd, ps, hd ** -0.5, window, got)
            torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
            outs.append(got)
    finally:
        lib.ie_set_decode_pair(ops.decode_cluster_max)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    ops.check_errors()


@pytest.mark.parametrize("nh,nkv,hd,ps", [(32, 8, 64, 16), (8, 2, 128, 16), (7, 1, 48, 8), (5, 5, 80, 4), (16, 2, 32, 16),
                                          (6, 3, 16, 16)])
@pytest.mark.parametrize("window", [0, 300])
@pytest.mark.parametrize("by_length", ["0", "1"])
def test_decode_attention_with_keys_as_the_rows_of_the_products(ops, nh, nkv, hd, ps, window, by_length, monkeypatch):
    """Requests of at most 8 rows (tokens x query heads per key/value head) run the decode
    kernels with the products swapped (keys are the instruction's rows); requests of 9 to 16 rows
    keep the 16-row layout, in the same launch.  Both layouts give the plain attention's result
    and differ from each other by rounding only (the order of 32-bit sums); a far key per
    request stands out, so that a key or a row in the wrong place shows.  Contexts from one key
    to thousands, at tile and page edges; portions of one to eight tokens, whose rows see
    different last keys."""
    group = nh // nkv
    ctx_lens = [1, 2, 15, 16, 17, 31, 32, 33, 63, 64, 65, 257, 1000, 2049, 3000, 8, 640, 96]
    q_lens = [min(1 + i % 8, c, max(1, 16 // group)) for i, c in enumerate(ctx_lens)]
    assert any(ql * group <= 8 for ql in q_lens)
    spike = [max(0, c - ql - window // 2) if window else (c - ql) // 3 for c, ql in zip(ctx_lens, q_lens)]
    monkeypatch.setattr(ops, "decode_balanced", by_length)
    q, k, v, tables, ctx = _attention_case(nh, nkv, hd, ps, q_lens, ctx_lens, torch.bfloat16, seed=13, spike=spike)
    want = torch.empty_like(q)
    RefOps().paged_attention(q, k, v, tables, ctx, nh, nkv, hd, ps, hd ** -0.5, window, want)
    lib = ops._attention_lib(hd)
    outs = []
    try:
        for narrow in (1, 0):
            lib.ie_set_decode_narrow(narrow)
            got = torch.zeros_like(q)
            ops.paged_attention(q, k, v, tables, ctx, nh, nkv, hd, ps, hd ** -0.5, window, got)
            torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
            outs.append(got)
    finally:
        lib.ie_set_decode_narrow(1 if ops.decode_narrow else 0)
    # one rounding step of bfloat16 at most between the layouts
    torch.testing.assert_close(outs[0].float(), outs[1].float(), atol=4e-3, rtol=8e-3)
    ops.check_errors()


@pytest.mark.parametrize("nh,nkv,hd,ps", [(32, 8, 64, 16), (8, 2, 128, 16), (4, 1, 64, 8)])
@pytest.mark.parametrize("window", [0, 1000])
@pytest.mark.parametrize("q_lens,ctx_lens", [([200], [3000]), ([130, 1, 260], [2600, 900, 260]), ([17], [1100])])
def test_prefill_attention_shares_the_keys_of_few_tiles_among_blocks(ops, nh, nkv, hd, ps, window, q_lens, ctx_lens):
    """A short portion at the end of a long prompt: too few query tiles to fill the GPU, so the
    keys of every tile are shared among several blocks and merged (head sizes 64 and 128).  One
    far key per request stands out; the result is the same with and without the sharing."""
    spike = [min(c - q, max(0, c - q - window // 2) if window else (c - q) // 3) for c, q in zip(ctx_lens, q_lens)]
    q, k, v, tables, ctx = _attention_case(nh, nkv, hd, ps, q_lens, ctx_lens, torch.bfloat16, seed=21, spike=spike)
    want = torch.empty_like(q)
    RefOps().paged_attention(q, k, v, tables, ctx, nh, nkv, hd, ps, hd ** -0.5, window, want)
    outs = []
    for share in (True, False):
        ops.prefill_key_splits = share
        try:
            got = torch.zeros_like(q)
            ops.paged_attention(q, k, v, tables, ctx, nh, nkv, hd, ps, hd ** -0.5, window, got)
            ctx._attention_plans = None
        finally:
            ops.prefill_key_splits = True
        torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
        outs.append(got)
    torch.testing.assert_close(outs[0].float(), outs[1].float(), atol=1e-2, rtol=1e-2)
    ops.check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,ps", [(32, 8, 64, 16), (3, 1, 32, 8), (8, 2, 128, 16)])
def test_paged_attention_finds_one_far_key(ops, dtype, nh, nkv, hd, ps):
    """Among hundreds of keys one stands out: at a page's first and last slot, in the first
    page, deep in the middle, and at the query's own position."""
    q_lens, ctx_lens = [1, 1, 1, 9, 1], [700, 513, 640, 300, 257]
    spike = [3, ps - 1, 511, 289, 256]
    q, k, v, tables, ctx = _attention_case(nh, nkv, hd, ps, q_lens, ctx_lens, dtype, seed=1, spike=spike)
    got = torch.empty_like(q)
    ops.paged_attention(q, k, v, tables, ctx, nh, nkv, hd, ps, hd ** -0.5, 0, got)
    want = torch.empty_like(q)
    RefOps().paged_attention(q, k, v, tables, ctx, nh, nkv, hd, ps, hd ** -0.5, 0, want)
    tol = dict(atol=2e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(got.float(), want.float(), **tol)
    # and the answer really is that key's value (for queries that can see it)
    seqs, pos = ctx.seq_of_token.tolist(), ctx.positions.tolist()
    for t in range(ctx.num_tokens):
        i = seqs[t]
        if pos[t] < spike[i]:
            continue
        page, off = int(tables[i, spike[i] // ps]), spike[i] % ps
        expect = v[page, :, off].float().repeat_interleave(nh // nkv, dim=0).reshape(-1)
        torch.testing.assert_close(got[t].float(), expect, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_window_edge(ops, dtype):
    """The key just inside the window counts, the one just outside does not."""
    nh, nkv, hd, ps, window = 4, 2, 32, 8, 24
    for key_pos, visible in ((100 - window + 1, True), (100 - window, False)):
        q, k, v, tables, ctx = _attention_case(nh, nkv, hd, ps, [1], [101], dtype, seed=2, spike=[key_pos])
        got = torch.empty_like(q)
        ops.paged_attention(q, k, v, tables, ctx, nh, nkv, hd, ps, hd ** -0.5, window, got)
        page, off = int(tables[0, key_pos // ps]), key_pos % ps
        expect = v[page, :, off].float().repeat_interleave(nh // nkv, dim=0).reshape(-1)
        close = torch.allclose(got[0].float(), expect, atol=3e-2, rtol=3e-2)
        assert close == visible
        want = torch.empty_like(q)
        RefOps().paged_attention(q, k, v, tables, ctx, nh, nkv, hd, ps, hd ** -0.5, window, want)
        torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)


def test_attention_refuses_a_head_size_it_cannot_take(ops):
    from inference_engine_b200.kernels import KernelError

    q, k, v, tables, ctx = _attention_case(2, 1, 16, 8, [1], [9], torch.float32)
    with pytest.raises(KernelError, match="head_dim"):
        ops.paged_attention(q, k, v, tables, ctx, 2, 1, 20, 8, 1.0, 0, torch.empty_like(q))
