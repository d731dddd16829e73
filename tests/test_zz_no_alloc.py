"""`ie_attention_decode_static`: the decode attention for hosts that may not allocate device
memory where they call it (a plugin inside a runtime that owns all device memory, a loop
whose owner forbids allocator calls).  It keeps its split partials in an array that is part
of the library instead of asking the caller for scratch.

The test calls the exported C symbol directly, twice in a row with different inputs (the
second call finds the array as the first left it), and compares with the regular entry point
`ie_attention_decode`, which gets scratch from the caller, and with the plain PyTorch attention
of `tests/ref_ops.py`, which shares no code with either.  The device's free memory as the
driver reports it (not torch's allocator, which an allocation inside the C function would
bypass) must be the same before and after the calls.  It also checks that a call whose partials
would not fit the built-in array is refused with a message and launches nothing.
This file sorts last on purpose, so a run that stops at the first failure has already run
every other test.
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

HD, NH, NKV, PAGE = 64, 32, 8, 16
TOO_SMALL = -1001


def _library():
    from inference_engine_b200.kernels.build import build_attention

    lib = ctypes.CDLL(str(build_attention(HD)))
    P, I, F = c_void_p, c_int, c_float
    lib.ie_attention_decode.argtypes = [P, P, P, P, I, P, P, P, P, P, I, I, I, I, I, F, I, I, P, P]
    lib.ie_attention_decode_static.argtypes = [P, P, P, P, I, P, P, P, I, I, I, I, I, F, I, I, P, P, c_char_p, I]
    lib.ie_attention_decode_scratch_floats.argtypes = [I, I, I]
    lib.ie_attention_decode_scratch_floats.restype = ctypes.c_longlong
    lib.ie_attention_decode_static_capacity_floats.restype = ctypes.c_longlong
    return lib


def _plain_attention(q, k, v, tables, ctx_lens):
    """What the entry point computes, by the plain PyTorch stand-in of the attention kernels."""
    import types

    from tests.ref_ops import RefOps

    b = len(ctx_lens)
    ctx = types.SimpleNamespace(
        num_tokens=b, num_seqs=b,
        positions=torch.tensor([c - 1 for c in ctx_lens], dtype=torch.int32, device="cuda"),
        seq_of_token=torch.arange(b, dtype=torch.int32, device="cuda"))
    out = torch.empty_like(q)
    RefOps().paged_attention(q, k, v, tables, ctx, NH, NKV, HD, PAGE, HD ** -0.5, 0, out)
    return out


def _case(ctx_lens, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    b = len(ctx_lens)
    pages_per = [-(-c // PAGE) for c in ctx_lens]
    total = sum(pages_per) + 2
    perm = torch.randperm(total, device="cuda", generator=g).to(torch.int32)
    tables = torch.full((b, max(pages_per)), -1, dtype=torch.int32, device="cuda")
    cursor = 0
    for i, n in enumerate(pages_per):
        tables[i, :n] = perm[cursor:cursor + n]
        cursor += n
    k = torch.randn(total, NKV, PAGE, HD, device="cuda", generator=g).bfloat16()
    v = torch.randn(total, NKV, PAGE, HD, device="cuda", generator=g).bfloat16()
    q = torch.randn(b, NH * HD, device="cuda", generator=g).bfloat16()
    cu_q = torch.arange(b + 1, dtype=torch.int32, device="cuda")
    ctx = torch.tensor(ctx_lens, dtype=torch.int32, device="cuda")
    return q, k, v, tables, cu_q, ctx


def test_static_scratch_entry_point_matches_the_regular_one_twice_in_a_row():
    lib = _library()
    stream = torch.cuda.current_stream().cuda_stream
    err = torch.zeros(4, dtype=torch.int32, device="cuda")
    msg = ctypes.create_string_buffer(512)
    splits = 5
    for call, ctx_lens in enumerate(([1000, 17, 333, 64, 1, 2048], [700, 900, 5])):
        q, k, v, tables, cu_q, ctx = _case(ctx_lens, seed=10 + call)
        b = len(ctx_lens)
        floats = lib.ie_attention_decode_scratch_floats(b, NKV, splits)
        assert 0 < floats <= lib.ie_attention_decode_static_capacity_floats()
        scratch = torch.empty(floats, dtype=torch.float32, device="cuda")
        tickets = torch.zeros(b * NKV, dtype=torch.int32, device="cuda")
        want = torch.zeros_like(q)
        rc = lib.ie_attention_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), tables.data_ptr(),
                                     tables.shape[1], cu_q.data_ptr(), ctx.data_ptr(), want.data_ptr(),
                                     scratch.data_ptr(), tickets.data_ptr(), b, NH, NKV, PAGE, k.shape[0], HD ** -0.5, 0,
                                     splits, err.data_ptr(), stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert not tickets.any()  # the launch left its counters at zero
        plain = _plain_attention(q, k, v, tables, ctx_lens)
        got = torch.zeros_like(q)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before, _ = torch.cuda.mem_get_info()
        rc = lib.ie_attention_decode_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), tables.data_ptr(),
                                            tables.shape[1], cu_q.data_ptr(), ctx.data_ptr(), got.data_ptr(),
                                            b, NH, NKV, PAGE, k.shape[0], HD ** -0.5, 0, splits,
                                            err.data_ptr(), stream, msg, len(msg))
        assert rc == 0, msg.value.decode()
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_before, "the device's free memory changed across the call"
        assert torch.cuda.memory_allocated() == before
        assert err.tolist()[0] == 0
        assert bool(got.float().abs().sum() > 0)
        torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
        torch.testing.assert_close(got.float(), plain.float(), atol=2e-2, rtol=2e-2)


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    lib = _library()
    q, k, v, tables, cu_q, ctx = _case([40, 50], seed=3)
    out = torch.full_like(q, 7.0)
    msg = ctypes.create_string_buffer(512)
    # pretend to bring 4096 requests at 32 splits: far beyond the built-in array
    rc = lib.ie_attention_decode_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), tables.data_ptr(),
                                        tables.shape[1], cu_q.data_ptr(), ctx.data_ptr(), out.data_ptr(),
                                        4096, NH, NKV, PAGE, k.shape[0], HD ** -0.5, 0, 32, None,
                                        torch.cuda.current_stream().cuda_stream, msg, len(msg))
    assert rc == TOO_SMALL
    text = msg.value.decode()
    assert "floats of scratch" in text and "built-in array holds" in text
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())  # nothing was launched
