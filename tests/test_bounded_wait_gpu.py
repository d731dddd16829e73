"""A wait inside a kernel that runs out: reported, tensor memory given back, context usable.

Every wait of the TMA-fed kernels on an mbarrier is bounded.  The product library's bound is
tenths of a second and nothing in a healthy run reaches it, so the way out of a failed wait is
exercised with the self-test build of the same sources (`kernels/build.py: build_selftest`):
256 polls, and a switch that makes every block tell a barrier to expect a copy which it then
does not ask for.  The wait gives up by construction; nothing spins without a limit, nothing
faults, and no copy is in flight when the block returns.
"""

from __future__ import annotations

import ctypes
from ctypes import c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
TIMEOUT = 5


@pytest.fixture(scope="module")
def selftest():
    from inference_engine_b200.kernels.build import build_selftest

    lib = ctypes.CDLL(str(build_selftest()))
    P, I = c_void_p, c_int
    for name in ("ie_gemm_tma_bf16", "ie_gemm_tc5_bf16"):
        getattr(lib, name).argtypes = [P, P, P, I, I, I, I, I, I, P, P]
    return lib


@pytest.mark.parametrize("kernel,m", [("tc5", 40), ("tma", 5)])
def test_a_wait_that_runs_out_is_reported_and_the_next_launch_is_right(selftest, kernel, m):
    from inference_engine_b200.kernels import get_ops
    from inference_engine_b200.kernels.cuda_ops import KernelError

    ops = get_ops("cuda")
    n, k, kblocks, splits = 1024, 2048, 8, 4  # 8 feature tiles x 4 slices of k: 32 blocks
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(m, k, device="cuda", generator=g).bfloat16()
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.05).bfloat16()
    want = x.double() @ w.double().t()
    err = torch.zeros(4, dtype=torch.int32, device="cuda")
    launch = getattr(selftest, f"ie_gemm_{kernel}_bf16")
    starve = getattr(selftest, f"ie_test_starve_{kernel}")
    stream = torch.cuda.current_stream().cuda_stream

    def product():
        out = torch.zeros(splits, m, n, device="cuda")
        rc = launch(x.data_ptr(), w.data_ptr(), out.data_ptr(), 0, m, n, k, kblocks, splits,
                    err.data_ptr(), stream)
        assert rc == 0
        torch.cuda.synchronize()  # returns: the kernel left by itself
        return out.sum(0).double()

    # healthy, with the short limit: no wait of a normal run comes near 256 polls
    torch.testing.assert_close(product(), want, atol=2e-4 * k ** 0.5, rtol=1e-5)
    assert err.tolist()[0] == 0
    # every block is told to expect a copy that never comes
    assert starve(1) == 0
    try:
        starved = product()
    finally:
        assert starve(0) == 0
    code, block_x, block_y, _ = err.tolist()
    assert code == TIMEOUT and 0 <= block_x < n // 128 and 0 <= block_y < splits
    assert not torch.allclose(starved, want, atol=1e-2)  # the result is not to be used
    ops.err.copy_(err)
    with pytest.raises(KernelError, match="bounded wait inside a kernel ran out"):
        ops.check_errors()
    assert ops.err.tolist()[0] == 0  # reported once, cleared
    # the context is whole: the same launch is right again (its tensor memory was given back,
    # or this one would find none), twice, and so is the library that serves generation
    err.zero_()
    for _ in range(2):
        torch.testing.assert_close(product(), want, atol=2e-4 * k ** 0.5, rtol=1e-5)
    assert err.tolist()[0] == 0
    out = torch.empty(m, n, device="cuda")
    ops.linear(x, w, out)
    torch.testing.assert_close(out.double(), want, atol=2e-4 * k ** 0.5, rtol=1e-5)
    ops.check_errors()
