"""The engine's kernels as Python calls on torch tensors.

Each method hands raw device pointers and the current CUDA stream to a plain-C function of
the in-tree shared library (``ctypes``; nothing is allocated on the way).  There is no
fallback: if the library cannot be built or loaded, or a tensor is not on a CUDA device,
the call raises.  Matrix products in bfloat16 go to the vendor library through ``torch.mm``
(the reference uses cuBLAS for them through ``nn.Linear``, engine/model/layers.py:126-129);
32-bit matrix products, attention, norms, rotary encoding, the cache write, the activation,
the embedding gather and sampling are the kernels under ``csrc/``.
"""

from __future__ import annotations

import contextlib
import ctypes
import functools
import os
from ctypes import c_float, c_int, c_void_p

from .build import ATTENTION_HEAD_DIMS, build_attention, build_core

_ERRORS = {
    1: "a token id outside the vocabulary",
    2: "a page or slot outside the cache",
    3: "a position outside the rotary table",
    4: "a block-table entry that was already given back",
    5: "a bounded wait inside a kernel ran out (a copy never arrived)",
}


class KernelError(RuntimeError):
    pass


class KernelTimer:
    """Device time per kind of kernel, from CUDA events recorded around every launch made while
    the timer is active (``with ops.timed() as timer``).  The events sit between the kernels,
    so a kernel's start-up no longer overlaps its predecessor: the sum is a little more than
    the step takes untimed; the shares are what it is for."""

    def __init__(self, torch) -> None:
        self.torch = torch
        self.spans: list[tuple[str, object, object]] = []

    def begin(self, name: str):
        start = self.torch.cuda.Event(enable_timing=True)
        start.record()
        return name, start

    def end(self, span) -> None:
        stop = self.torch.cuda.Event(enable_timing=True)
        stop.record()
        self.spans.append((span[0], span[1], stop))

    def summary(self) -> dict[str, dict]:
        """kind -> {"launches": n, "ms": total device time}; waits for the device."""
        self.torch.cuda.synchronize()
        out: dict[str, dict] = {}
        for name, start, stop in self.spans:
            row = out.setdefault(name, {"launches": 0, "ms": 0.0})
            row["launches"] += 1
            row["ms"] += start.elapsed_time(stop)
        return out


def _kind(name):
    """Marks a kernel method with the kind its launches are counted under by a KernelTimer and
    shown under in a profiler's timeline (NVTX ranges, with IE_B200_NVTX=1).  ``name`` is a
    string or a function of the call's keyword arguments."""
    def decorate(method):
        def call(self, *args, **kwargs):
            timer, nvtx, recorder = self._timer, self.nvtx, self._recorder
            if timer is None and not nvtx and recorder is None:
                return method(self, *args, **kwargs)
            label = name if isinstance(name, str) else name(kwargs)
            if recorder is not None:
                recorder.append((label, functools.partial(method, self, *args, **kwargs)))
            if nvtx:
                self.torch.cuda.nvtx.range_push(label)
            span = timer.begin(label) if timer is not None else None
            try:
                return method(self, *args, **kwargs)
            finally:
                if span is not None:
                    timer.end(span)
                if nvtx:
                    self.torch.cuda.nvtx.range_pop()
        call.__name__, call.__doc__ = method.__name__, method.__doc__
        return call
    return decorate


def _dtype_code(t) -> int:
    import torch

    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {t.dtype}")


class CudaOps:
    name = "cuda-sm100a"

    def __init__(self, device="cuda") -> None:
        import torch

        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: the engine has no CPU path")
        self.torch = torch
        self.device = torch.device(device)
        self.lib_path = build_core()
        try:
            self.lib = ctypes.CDLL(str(self.lib_path))
        except OSError as exc:
            raise KernelError(f"the kernel library {self.lib_path} could not be loaded: {exc}") from exc
        self._declare()
        # programmatic dependent launch between the engine's own kernels (IE_B200_PDL=0: off)
        self.pdl = os.environ.get("IE_B200_PDL", "1") != "0"
        self.lib.ie_set_pdl(1 if self.pdl else 0)
        self.err = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._err_ptr = self.err.data_ptr()
        self._attn_libs: dict[int, object] = {}
        self._argmax_scratch = None
        self._tickets = None
        self._retired_tickets = []
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.attn_tc5 = os.environ.get("IE_B200_ATTN_TC5", "1") != "0"  # tcgen05 prefill attention
        self.prefill_key_splits = os.environ.get("IE_B200_PREFILL_KEY_SPLITS", "1") != "0"
        # up to this many query tiles x heads per SM a block takes two tiles of a request (a late and an early one)
        self.prefill_paired_max = float(os.environ.get("IE_B200_PREFILL_PAIRED_MAX", 4))
        # the decode kernel cuts contexts until about this many blocks run (one block per SM)
        self.decode_split_target = int(os.environ.get("IE_B200_DECODE_SPLIT_TARGET", 128))
        # up to this many parts of a context merge inside a thread-block cluster (2, 4, 8; 0: never),
        # for steps whose block tables hold at most `decode_cluster_tokens` tokens per request
        self.decode_cluster_max = int(os.environ.get("IE_B200_DECODE_PAIR", 8))
        self.decode_cluster_tokens = int(os.environ.get("IE_B200_DECODE_CLUSTER_TOKENS", 4096))
        # requests with at most 8 rows (tokens x query heads per key/value head) run the decode
        # kernels' swapped products: keys are the instruction's rows ("0": the 16-row layout for all)
        self.decode_narrow = os.environ.get("IE_B200_DECODE_NARROW", "1") != "0"
        # batches whose contexts differ much in length go to the decode kernel that deals key tiles
        # by length ("auto": when the step's context says so; "1": always; "0": never)
        self.decode_balanced = os.environ.get("IE_B200_DECODE_BALANCED", "auto")
        self.decode_balanced_blocks_per_pair = 32
        # by-request decode attention in two-warp blocks where that saves a round ("0": never)
        # ("2", "3": always blocks of as many warps when there are more blocks than SMs, for comparisons)
        small = os.environ.get("IE_B200_DECODE_SMALL", "1")
        self.decode_small = small != "0"
        self._force_small = int(small) if small in ("2", "3") else 0
        self._small_per_sm: dict[tuple[int, int], int] = {}
        self._dealing_look, self._dealing_answer = None, 0  # the last batch decode_dealing looked at, and its answer
        self.balanced_launches = 0
        # which kernel takes few-row bfloat16 products: "tma" (the TMA-fed weight-streaming kernel)
        # or "lib" (the vendor library, for comparisons)
        self.few_row_gemm = os.environ.get("IE_B200_FEW_ROW_GEMM", "tma")
        # ... up to this many 128-feature tiles (measured on the 1B shape: up to 8 rows the kernel
        # streams 67 MB in 12.0 us where the vendor library takes 12.7, and the 525 MB of the
        # head in 82 us against 79.5; from 9 rows on its second column tile makes it slower on
        # wide matrices, so only those that must be cut along k to fill the GPU go to it)
        self.tma_max_tiles = int(os.environ.get("IE_B200_TMA_MAX_TILES", 256))
        self.tma_max_tiles_wide = min(self.tma_max_tiles, self.sm_count // 2)  # 9 to 16 rows
        self.tma_max_blocks = int(os.environ.get("IE_B200_TMA_MAX_BLOCKS", 3 * self.sm_count // 2))
        # Products of 17 to `batch_gemm_rows` rows with a long inner dimension: the tcgen05
        # weight-streaming kernel (IE_B200_BATCH_GEMM=0: the vendor library).  Measured on the 1B
        # shape at 64 rows: the down projection (K = 8192) 11.0 us against the library's 13.0,
        # but QKV, output and gate-up (K = 2048) 7.3 / 6.3 / 16.3 against 5.7 / 5.5 / 13.5: every
        # block copies all tokens' activations through its SM's copy engine beside the weights,
        # which the library's kernels share within a cluster.  So only long inner dimensions, and
        # only where its blocks (feature tiles x cuts along k) fit the SMs in one round: at the 3B
        # shape the down projection (3072 x 8192) 13.5 against 14.2 us, at the 8B shape (4096 x
        # 14336: 224 blocks) 33.6 against 25.4, and its K = 4096 products 13 to 45 % behind.
        # the gated feed-forward's first product with the activation in its kernel (IE_B200_GATED_GEMM=0: off)
        self.gated_gemm = os.environ.get("IE_B200_GATED_GEMM", "1") != "0"
        # products of more than a few rows whose output is so narrow that the library's kernel would
        # leave most SMs idle are cut along the inner dimension and run as one strided batched product
        # (the parts are added by the consumer, like those of the few-row kernel)
        self.blas_split_k = os.environ.get("IE_B200_BLAS_SPLIT_K", "1") != "0"
        self.batch_gemm = os.environ.get("IE_B200_BATCH_GEMM", "1") != "0"
        self.batch_gemm_rows = int(os.environ.get("IE_B200_BATCH_GEMM_ROWS", 64))
        self.batch_gemm_max_tiles = int(os.environ.get("IE_B200_BATCH_GEMM_MAX_TILES", 256))
        self.batch_gemm_min_k = int(os.environ.get("IE_B200_BATCH_GEMM_MIN_K", 8192))
        # only where the kernel's blocks fit the SMs in one round
        self.batch_gemm_one_round = os.environ.get("IE_B200_BATCH_GEMM_ONE_ROUND", "1") != "0"
        self._device_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self._raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
        self._timer: KernelTimer | None = None
        self._recorder: list | None = None
        self.nvtx = os.environ.get("IE_B200_NVTX", "0") == "1"  # an NVTX range around every kernel call
        self.launches = 0  # launches of this library's kernels (library matrix products not counted)
        self.launch_counts: dict[str, int] = {}  # the same, per kernel
        self._cluster_fit: dict[tuple[int, int], int] = {}  # (head size, parts) -> clusters the device runs at once

    def _declare(self) -> None:
        P, I, F, L = c_void_p, c_int, c_float, ctypes.c_longlong
        sigs = {
            "ie_embedding": [P, I, P, P, I, I, I, P, P],
            "ie_rmsnorm": [P, P, I, L, P, F, P, I, P, I, I, P],
            "ie_rope_kv_write": [P, I, L, P, P, I, I, P, P, P, I, P, I, I, I, I, I, I, P, P],
            "ie_silu_mul": [P, I, I, L, P, I, I, I, I, P],
            "ie_gemm_tma_gated_bf16": [P, P, P, I, I, I, P, P],
            "ie_argmax": [P, I, I, I, P, P, P],
            "ie_gemm_f32": [P, P, P, I, I, I, P],
            "ie_gemm_tma_bf16": [P, P, P, I, I, I, I, I, I, P, P],
            "ie_gemm_tc5_bf16": [P, P, P, I, I, I, I, I, I, P, P],
            "ie_gemm_tc5_ok": [I, I, I],
            "ie_paged_attention_generic": [P, P, P, I, P, I, P, P, P, I, I, I, I, I, I, F, I, P, P],
            "ie_sample": [P, I, I, P, P, P, P, P, P, I, P, P, P, P, P],
        }
        for name, args in sigs.items():
            fn = getattr(self.lib, name)
            fn.argtypes, fn.restype = args, c_int
            setattr(self, "_" + name[3:], fn)

    # --- helpers ----------------------------------------------------------------------------

    def _stream(self) -> int:
        """The raw handle of torch's current stream on this device (asked on every launch, so
        through the cheap accessor when torch has it)."""
        if self._raw_stream is not None:
            return self._raw_stream(self._device_index)
        return self.torch.cuda.current_stream(self.device).cuda_stream

    def _check(self, code: int, what: str) -> None:
        self.launches += 1
        self.launch_counts[what] = self.launch_counts.get(what, 0) + 1
        if code != 0:
            raise KernelError(f"{what}: CUDA error {code} at launch")

    @staticmethod
    def _ptr(t) -> int | None:
        return None if t is None else t.data_ptr()

    def check_errors(self) -> None:
        """Read the device error word (this waits for the stream) and raise if a kernel saw
        an index out of range or gave up a wait."""
        self.raise_reported(self.err.tolist())

    def raise_reported(self, words) -> None:
        """``words``: a copy of the error word (code, value, where, spare).  A non-zero code
        clears the word on the device (the first report wins, so the next fault must find it
        empty) and raises."""
        code, value, where = words[:3]
        if code:
            self.err.zero_()
            raise KernelError(f"kernel check failed: {_ERRORS.get(code, code)} "
                              f"(value {value}, at row/token {where})")

    @contextlib.contextmanager
    def timed(self, lead_ms: float = 0.0):
        """``with ops.timed() as timer: ...; timer.summary()``: CUDA-event time per kind of kernel
        for everything launched inside the block (eager launches only: a replayed capture is one
        launch).  The host launches small kernels more slowly than the device runs them, and an
        event pair around a kernel that has not been launched yet measures the host; with
        ``lead_ms`` the device is first kept busy that long, so that the block's launches queue
        up behind it and the events see device time only."""
        timer = KernelTimer(self.torch)
        if lead_ms > 0:
            self.busy_wait(lead_ms)
        self._timer = timer
        try:
            yield timer
        finally:
            self._timer = None

    @contextlib.contextmanager
    def recording(self):
        """``with ops.recording() as calls``: every kernel call made inside the block is also kept
        as ``(kind, callable)``; calling the callable launches the same kernel on the same
        tensors again (for timing one kind of kernel by itself, back to back over a step's
        layers)."""
        calls: list = []
        self._recorder = calls
        try:
            yield calls
        finally:
            self._recorder = None

    def busy_wait(self, ms: float) -> None:
        """Keep the device busy for about ``ms``, so that what the host launches next queues up."""
        khz = self.torch.cuda.get_device_properties(self.device).clock_rate
        self.torch.cuda._sleep(int(ms * khz))

    # --- kernels ----------------------------------------------------------------------------

    @_kind("embedding")
    def embedding(self, table, ids, out) -> None:
        self._check(self._embedding(table.data_ptr(), _dtype_code(table), ids.data_ptr(),
                                    out.data_ptr(), ids.shape[0], table.shape[1], table.shape[0],
                                    self._err_ptr, self._stream()), "embedding")

    @staticmethod
    def _partials(t) -> tuple[int, int]:
        """A 3-D tensor ``[S, rows, cols]`` stands for the sum of its S slices (the parts of a
        matrix product split along the inner dimension): (S, elements between slices)."""
        if t is None or t.dim() == 2:
            return 1, 0
        return t.shape[0], t.stride(0)

    @_kind("norm")
    def rmsnorm(self, h, delta, weight, eps, out, rows=None) -> None:
        n = h.shape[0] if rows is None else rows.shape[0]
        parts, stride = self._partials(delta)
        self._check(self._rmsnorm(h.data_ptr(), self._ptr(delta), parts, stride, weight.data_ptr(), eps,
                                  out.data_ptr(), _dtype_code(out), self._ptr(rows), n,
                                  h.shape[1], self._stream()), "rmsnorm")

    FEW_ROWS = 16  # up to this many rows a bfloat16 product runs the weight-streaming kernel

    def tma_split(self, n_out: int, k: int) -> tuple[int, int]:
        """(64-wide k blocks per split, splits) for the TMA-fed few-row product: one block of
        128 features per SM if there are enough features, else the inner dimension is cut so
        that about every SM has a block; a block takes at most 32 k blocks."""
        tiles = -(-n_out // 128)
        total = -(-k // 64)
        splits = max(1, min(total, self.sm_count // tiles))
        per = min(-(-total // splits), 32)
        # one copy brings up to four k blocks when they divide the slice: round the slice up to
        # a multiple of 4 (or 2) unless that leaves many SMs without a block
        for multiple in (4, 2):
            rounded = min(-(-per // multiple) * multiple, 32)
            if rounded != per and -(-total // rounded) * tiles * 10 >= -(-total // per) * tiles * 8:
                per = rounded
                break
            if rounded == per:
                break
        return per, -(-total // per)

    def blas_split(self, m: int, n: int, k: int) -> int:
        """Into how many parts along the inner dimension a bfloat16 product of ``m`` rows is cut before
        it goes to the library (1: not at all).  The library's kernels take about 128 x 128 outputs per
        block and do not cut the inner dimension themselves: the 64-row down projection of the 1B shape
        runs as 16 blocks on 148 SMs, 13 us where its 33.5 MB would stream in 5.  As a batched product
        over 8 slices of k it takes 8.5 us (measured, 1B shape, us: down at 17 / 64 / 256 / 512 rows
        13.0 / 13.2 / 13.8 / 18.9 -> 8.1 / 8.5 / 10.6 / 15.4; output projection at 17 / 64 rows 5.6 / 5.8
        -> 4.4 / 4.8; QKV 5.8 -> 5.0; products with many output features, gate-up and the head, lose).
        A power of two: at most 8 up to 32 rows, 4 up to 256, 2 up to 512 (the parts' sums are written and
        read again: 96 rows of the down projection take 9.6 us in 8 parts, 8.6 in 4); no more parts than
        bring the library's blocks to about 1.2 per SM; slices of at least 256.  The rule was set against
        `profile_gemm`'s tables of the 1B, 3B and 8B shapes' products at 9 to 512 rows: it is 0.6 %, 1.4 %
        and 1.8 % behind the best of 1, 2, 4, 8 parts on average, 4 %, 8 % and 15 % at worst."""
        if not self.blas_split_k or m > 512:
            return 1
        blocks = -(-m // 128) * -(-n // 128)
        parts = 1
        most = 8 if m <= 32 else 4 if m <= 256 else 2
        while parts * 2 <= min(1.2 * self.sm_count / blocks, most) and k % (parts * 2 * 64) == 0 and k // (parts * 2) >= 256:
            parts *= 2
        return parts

    @_kind(lambda kwargs: "linear:" + kwargs.get("tag", "linear"))
    def linear(self, x, w, out=None, *, ws=None, tag="linear", out_dtype=None, allow_split=False):
        """``x[M, K] @ w[N, K]^T``.  With ``out`` given the product is written there; otherwise a
        buffer named ``tag`` is taken from ``ws``.  With ``allow_split`` the result may come back
        as ``[S, M, N]`` partial sums (32-bit) that the consumer adds in order."""
        torch = self.torch
        m, k = x.shape
        n = w.shape[0]
        if out is not None:
            out_dtype = out.dtype
        if x.dtype == torch.float32:
            if out_dtype != torch.float32 or w.dtype != torch.float32:
                raise KernelError("the 32-bit matrix product takes and gives 32-bit tensors")
            if out is None:
                out = ws.buffer(tag, m, n, torch.float32)
            if m:
                self._check(self._gemm_f32(x.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k,
                                           self._stream()), "gemm_f32")
            return out
        # The weight-streaming kernel pays where the library leaves SMs idle: few output
        # features (fewer 16-feature blocks than SMs) and a long inner dimension to split.
        few_rows = 0 < m <= self.FEW_ROWS and k % 8 == 0 and x.is_contiguous() and w.is_contiguous()
        splittable = (allow_split and out is None and out_dtype == torch.float32 and m > 0
                      and x.is_contiguous() and w.is_contiguous())
        library_parts = self.blas_split(m, n, k) if splittable else 1
        if few_rows and m > 8 and library_parts > 1 and (k >= 4096 or n * k >= 12 << 20):
            # (9 to 16 rows, a long inner dimension or a large matrix: the batched library product is ahead,
            # 8.0 against 9.5 us on the 1B shape's down projection, 7.9 against 9.1 on the 3B shape's QKV)
            few_rows = False
        if (few_rows and self.few_row_gemm == "tma"
                and -(-n // 128) <= (self.tma_max_tiles if m <= 8 else self.tma_max_tiles_wide)):
            kbps, splits = self.tma_split(n, k) if allow_split and out is None else (-(-k // 64), 1)
            # (more than one and a half rounds of blocks over the SMs: the library's kernels are
            # ahead there, 41.8 against 45.7 us on the 8B shape's gate-up matrix)
            if kbps <= 32 and -(-n // 128) * splits <= self.tma_max_blocks:
                if splits > 1:
                    out = ws.buffer(tag, splits * m, n, torch.float32).view(splits, m, n)
                elif out is None:
                    out = ws.buffer(tag, m, n, out_dtype)
                self._check(self._gemm_tma_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), _dtype_code(out),
                                                m, n, k, kbps, splits, self._err_ptr, self._stream()), "gemm_tma")
                return out
        if library_parts > 1:
            parts, ks = library_parts, k // library_parts
            out = ws.buffer(tag, parts * m, n, torch.float32).view(parts, m, n)
            # slice p of the inner dimension: x[:, p ks : (p + 1) ks] and w[:, p ks : (p + 1) ks]^T, as views
            torch.bmm(x.view(m, parts, ks).permute(1, 0, 2), w.view(n, parts, ks).permute(1, 2, 0),
                      out_dtype=torch.float32, out=out)
            return out
        # A batch of decode tokens (17 to 256 rows): still a stream of weights; the tcgen05
        # kernel with the operands' roles swapped, cut along k like the few-row kernel.
        if (self.batch_gemm and self.FEW_ROWS < m <= self.batch_gemm_rows and x.is_contiguous()
                and w.is_contiguous() and self._gemm_tc5_ok(m, n, k)
                and -(-n // 128) <= self.batch_gemm_max_tiles and k >= self.batch_gemm_min_k
                and (not self.batch_gemm_one_round or (
                    allow_split and out is None and -(-n // 128) * self.tma_split(n, k)[1] <= self.sm_count))):
            per, splits = self.tma_split(n, k) if allow_split and out is None else (k // 64, 1)
            if splits > 1:
                out = ws.buffer(tag, splits * m, n, torch.float32).view(splits, m, n)
            elif out is None:
                out = ws.buffer(tag, m, n, out_dtype)
            self._check(self._gemm_tc5_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), _dtype_code(out),
                                            m, n, k, per, splits, self._err_ptr, self._stream()), "gemm_tc5")
            return out
        if out is None:
            out = ws.buffer(tag, m, n, out_dtype)
        if m == 0:
            return out
        if out.dtype == x.dtype:
            torch.mm(x, w.t(), out=out)
        else:
            torch.mm(x, w.t(), out_dtype=out.dtype, out=out)
        return out

    @_kind("rotary+cache")
    def rope_kv_write(self, qkv, positions, table, rotary_dim, q_out, k_cache, v_cache,
                      slot_mapping, nh, nkv, hd, page_size) -> None:
        if table is not None and table.shape[2] * 2 != rotary_dim:
            raise KernelError("rotary table does not match rotary_dim")
        if rotary_dim > hd or rotary_dim % 2:
            raise KernelError(f"rotary_dim {rotary_dim} must be even and at most head_dim {hd}")
        parts, stride = self._partials(qkv)
        self._check(self._rope_kv_write(
            qkv.data_ptr(), parts, stride, positions.data_ptr(), self._ptr(table), rotary_dim,
            0 if table is None else table.shape[0], q_out.data_ptr(), k_cache.data_ptr(),
            v_cache.data_ptr(), _dtype_code(q_out), self._ptr(slot_mapping), q_out.shape[0],
            nh, nkv, hd, page_size, k_cache.shape[0], self._err_ptr, self._stream()), "rope_kv_write")

    def _attention_lib(self, hd: int):
        """The tensor-core attention library for head size ``hd`` (built on first use)."""
        lib = self._attn_libs.get(hd)
        if lib is None:
            lib = ctypes.CDLL(str(build_attention(hd)))
            lib.ie_set_pdl(1 if self.pdl else 0)
            lib.ie_set_decode_pair(self.decode_cluster_max)
            lib.ie_set_decode_narrow(1 if self.decode_narrow else 0)
            P, I, F = c_void_p, c_int, c_float
            lib.ie_attention_decode.argtypes = [P, P, P, P, I, P, P, P, P, P, I, I, I, I, I, F, I, I, P, P]
            lib.ie_attention_prefill.argtypes = [P, P, P, P, I, P, P, P, I, I, I, I, I, I, F, I, P, P]
            lib.ie_attention_prefill_tc5.argtypes = [P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, I, F, I, I, P, P, P, P]
            lib.ie_attention_prefill_tc5_scratch_floats.argtypes = [I, I, I]
            lib.ie_attention_prefill_tc5_scratch_floats.restype = ctypes.c_longlong
            lib.ie_attention_prefill_tc5_ok.argtypes = [I, I]
            lib.ie_attention_decode_scratch_floats.argtypes = [I, I, I]
            lib.ie_attention_decode_scratch_floats.restype = ctypes.c_longlong
            lib.ie_attention_decode_balanced.argtypes = [P, P, P, P, I, P, P, P, P, P, I, I, I, I, I, F, I, I, P, P]
            lib.ie_attention_decode_ordered.argtypes = [P, P, P, P, I, P, P, P, P, P, I, I, I, I, I, F, I, I, P, I, P, P]
            lib.ie_attention_decode_balanced_scratch_floats.argtypes = [I, I, I]
            lib.ie_attention_decode_balanced_scratch_floats.restype = ctypes.c_longlong
            lib.ie_attention_decode_max_clusters.argtypes = [I]
            self._attn_libs[hd] = lib
        return lib

    def _decode_tickets(self, count: int):
        """Zeroed counters for the decode kernel's split merge; every launch leaves them zero."""
        if self._tickets is None or self._tickets.numel() < count:
            if self._tickets is not None:
                self._retired_tickets.append(self._tickets)  # captured launches may still point at it
            self._tickets = self.torch.zeros(max(count, 16384), dtype=self.torch.int32, device=self.device)
        return self._tickets

    def _clusters_at_once(self, hd: int, parts: int) -> int:
        """How many clusters of ``parts`` decode attention blocks the device runs at one time for
        head size ``hd`` (a cluster's blocks must find room in one group of SMs at the same
        time, so this is less than the SMs over ``parts``); 0: unknown."""
        key = (hd, parts)
        if key not in self._cluster_fit:
            self._cluster_fit[key] = int(self._attention_lib(hd).ie_attention_decode_max_clusters(parts))
        return self._cluster_fit[key]

    def decode_splits(self, num_seqs: int, nkv: int, table_tokens: int = 0, hd: int | None = None) -> int:
        """Into how many parts the decode kernel cuts each context.  One block per (request,
        key/value head) streams at an SM's full rate, so contexts are only cut when there are
        few such blocks (small batches).  2, 4 or 8 parts run as one thread-block cluster and
        merge through shared memory, which is worth more than the last few blocks: the count is
        rounded down to one of those (and to one of which the device runs all clusters at one
        time, if the head size ``hd`` is given), except for long contexts (``table_tokens``: what
        the step's block tables can hold), where as many parts as give nearly every SM a block
        stream faster, whichever way they merge.  The number depends on the batch and the tables'
        width alone, never on the contexts' lengths, so that a captured launch stays valid."""
        pairs = max(num_seqs * nkv, 1)
        if table_tokens > self.decode_cluster_tokens:
            # long contexts: a block for nearly every SM counts for more than the way the parts merge
            # (2 requests x 8 heads x 32,768 tokens: 9 parts 30.5 us, 8 parts 55, 4 parts 51)
            parts = max(1, min(self.sm_count // pairs, 16 if pairs >= 8 else 32))
            # blocks of four warps run two to an SM: where that fills the device much better than one
            # block of eight warps per SM (10 to 12 requests of 8 heads: 96 blocks for 148 SMs, or 288
            # for 296 slots), it is worth their dearer merge (12 x 8,192 tokens: 47 -> 42 us)
            halves = (2 * self.sm_count) // pairs
            if 1 < halves <= 32 and pairs * halves / (2 * self.sm_count) > 1.25 * pairs * parts / self.sm_count:
                parts = halves
            return parts
        parts = max(1, min(self.decode_split_target // pairs, 32))
        if self.decode_cluster_max < 2 or parts < 2:
            return parts
        parts = min(8 if parts >= 8 else 4 if parts >= 4 else 2, self.decode_cluster_max)
        # all clusters have to run at one time (16 clusters of 8 do not: a second round of blocks
        # doubled the kernel's time at batch 2); else the next smaller size
        while hd is not None and parts > 2 and 0 < self._clusters_at_once(hd, parts) < pairs:
            parts //= 2
        return parts

    BY_REQUEST, BY_LENGTH, SMALL_2, SMALL_3 = 0, 1, 2, 3  # how a decode step's attention is dealt (StepContext.ragged)

    def _decode_blocks_per_sm(self, hd: int, warps: int) -> int:
        key = (hd, warps)
        if key not in self._small_per_sm:
            self._small_per_sm[key] = int(self._attention_lib(hd).ie_attention_decode_blocks_per_sm(warps))
        return self._small_per_sm[key]

    @staticmethod
    def _by_request_estimate(by_length, at_once: int, scale: float, setup: float) -> float:
        """How long blocks dealt by request take, in tokens a four-warp block walks: ``by_length`` the
        contexts, the longest first, ``at_once`` of them on the device at one time, a block's time
        ``setup + scale * length``.  The requests beyond the first round start as those of the round
        before end, the shortest of them first."""
        if by_length[0] <= 1.1 * by_length[-1]:  # (about one length: whole rounds)
            return -(-len(by_length) // at_once) * (setup + scale * by_length[0])
        finish = []
        for i, n in enumerate(by_length):
            r, k = divmod(i, at_once)
            finish.append((finish[r * at_once - 1 - k] if r else 0.0) + setup + scale * n)
        return max(finish)

    def decode_dealing(self, ctx_lens, nkv: int, hd: int | None = None) -> int:
        """How the decode attention of a step over contexts of these lengths is dealt: key tiles by
        length (:meth:`decode_by_length`), or by request, and then in blocks of 3 or 2 warps (3 or 4 of
        them to an SM at head size 64, against 2 of the four-warp blocks) where the step's blocks then
        need fewer rounds over the device.  A block of w warps takes a set-up worth 300 tokens and
        4 / w of its context (in tokens a four-warp block walks; measured at 1,024 tokens: a round of
        four-warp blocks 13 us, of three-warp blocks 18, of two-warp blocks 24); the rounds are
        estimated by :meth:`_by_request_estimate`, and smaller blocks must be 7 % ahead.  Measured at
        head size 64, us per layer, four-warp blocks -> the choice: 40 requests x 1,024 tokens 25.8 ->
        17.9 (3 warps), 55 x 1,024 26.9 -> 19.6 (0.90 of the copy rate), 64 x 1,024 27.3 -> 24.8 (2 warps),
        80 x 1,024 40.0 -> 35.9 (3), 128 x 1,024 54.6 -> 49.4 (2), 160 x 1,024 68.1 -> 56.4 (3), 64 x 4,096
        96.4 -> 90.4, 64 x 256 10.4 -> 8.3, 40 of 768 to 1,280 tokens 22.1 -> 19.8; kept in four-warp blocks,
        the longest first: 48 of 512 to 1,536 tokens (19.5; 23.1 in three-warp blocks), 64 of 64 to 2,048
        (27.1; 43.6 in two-warp blocks)."""
        # (the answer is kept while the batch looks the same: as many contexts, the same longest and the
        # same sum, each to 64 tokens per request; the estimates cost 60 us at 64 requests, 220 at 256)
        count = len(ctx_lens)
        look = (count, nkv, hd, max(ctx_lens) >> 6 if count else 0, sum(ctx_lens) // (64 * max(count, 1)),
                self.decode_balanced, self.decode_small, self._force_small)
        if look == self._dealing_look:
            return self._dealing_answer
        self._dealing_look, self._dealing_answer = look, self._decode_dealing(ctx_lens, nkv, hd)
        return self._dealing_answer

    def _decode_dealing(self, ctx_lens, nkv: int, hd: int | None = None) -> int:
        dealt_by_length = self.decode_by_length(ctx_lens, nkv, hd)
        first = self.BY_LENGTH if dealt_by_length else self.BY_REQUEST
        if not self.decode_small or hd is None or hd not in ATTENTION_HEAD_DIMS or not ctx_lens:
            return first
        pairs = len(ctx_lens) * nkv
        if self._force_small and pairs > self.sm_count:
            return self._force_small
        usual = self._decode_blocks_per_sm(hd, 4)
        if pairs <= max(usual, 1) * self.sm_count or self.decode_balanced == "1":
            return first  # (one round of the usual blocks anyway; up to one block per SM: eight warps)
        by_length = sorted(ctx_lens, reverse=True)
        setup = 300.0
        best, best_time = self.BY_REQUEST, 0.93 * self._by_request_estimate(
            by_length, max(1, usual * self.sm_count // nkv), 1.0, setup)
        if dealt_by_length:  # (the smaller blocks then have to beat that kernel: 48 requests x 4,096 tokens
            # take 75.9 us dealt by length, 64.4 in three-warp blocks)
            best, best_time = self.BY_LENGTH, self._dealt_estimates(ctx_lens, nkv, hd)[1]
        for warps, code in ((3, self.SMALL_3), (2, self.SMALL_2)):
            per_sm = self._decode_blocks_per_sm(hd, warps)
            if per_sm <= usual:
                continue
            time = self._by_request_estimate(by_length, max(1, per_sm * self.sm_count // nkv), 4.0 / warps, setup)
            if time < best_time:
                best, best_time = code, time
        return best

    def _dealt_estimates(self, ctx_lens, nkv: int, hd: int | None = None) -> tuple[float, float]:
        """(dealt by request, dealt by length): how long the two decode attention kernels take for
        contexts of these lengths, in tokens one block walks (a block of eight warps up to one (request,
        head) pair per SM, of four warps, two to an SM, beyond).  By request the step lasts as long as
        the longest context over its splits (twice that where the splits make more blocks than SMs:
        those blocks have four warps; and a set-up more where they merge through memory), or the whole
        work over the blocks the device runs at once, if that is more.  By length: what that kernel's own
        dealing gives the slowest block (below).  Measured, us per
        layer, by request / by length, with the estimate's answer: 12 requests x 4,096 tokens 25.8 / 33.4
        (by request), 11 x 2,048 12.8 / 19.5 (by request), 7 x 32,768 98.7 / 85.9 (by length), 10 x 8,192
        41.0 / 36.4 (by length), 24 x 8,192 92.8 / 74.4 (by length), 28 x 8,192 94.3 / 85.6 (by length),
        32 x 8,192 95.4 / 97.0 (by request), 20 x 4,096 47.6 / 37.3 (by length), 24 x 4,096 48.0 / 41.9 (by
        length), 28 x 4,096 48.5 / 47.8 (by request), 24 x 2,048 25.4 / 35.0 (by request), 40 of 128 to
        2,048 tokens 26 / 34 (by request), 9 x 4,096 25.1 / 18.5 (by length: two pieces per pair, one
        round); 14 x 8,192 49.5 / 47.1 is answered by request."""
        pairs = len(ctx_lens) * nkv
        work = sum(ctx_lens) * nkv
        longest = max(ctx_lens)
        slots = self.sm_count if pairs <= self.sm_count else 2 * self.sm_count
        table_tokens = 1024  # (what the step's block tables hold: widths double from 64 pages of 16 tokens)
        while table_tokens < longest:
            table_tokens *= 2
        splits = self.decode_splits(len(ctx_lens), nkv, table_tokens, hd)
        # blocks run in rounds over the slots; the last round is as long as a block even when few
        # blocks are in it (40 requests x 8 heads of 4,096 tokens, 320 blocks on 296 slots: 93 us by
        # request, 65 us by length)
        if pairs <= self.sm_count:
            by_request = longest / splits
            if pairs * splits > self.sm_count:   # (the splits' blocks have four warps)
                by_request = 2 * by_request * -(-pairs * splits // (2 * self.sm_count))
            if splits not in (1, 2, 4, 8):       # (merged through memory by the block that ends last)
                by_request += 1536
            by_request = max(by_request, work / slots)
        else:
            rounds = pairs * splits / slots
            last_round = (-(-pairs * splits // slots) - rounds) * work / (pairs * splits)
            by_request = max(longest / splits, work / slots + last_round)
        # By length, as that kernel deals (attention_mma.cu): every pair's tiles in pieces of about an
        # even share, dealt in rounds over the blocks, or, where the pieces would leave the slowest block
        # well behind, equal ranges of the list of all tiles, which lie in 1 + pairs / blocks stretches
        # of different pairs on average.  A piece or stretch costs six tiles per warp to set up.
        warps, keys = (8 if pairs <= self.sm_count else 4), (32 if hd is None or hd <= 64 else 16)  # (keys per tile)
        tiles = [-(-c // keys) for c in ctx_lens]
        share = max(-(-sum(tiles) * nkv // slots), warps)
        pieces = [max(1, min((n + share // 2) // share, n // warps)) for n in tiles]
        largest = max(-(-n // k) for n, k in zip(tiles, pieces))
        piece_rounds = -(-sum(pieces) * nkv // slots)
        setup = 6 * warps
        if piece_rounds * largest > share + setup:
            by_length = share + setup * (1 + pairs / slots)
        else:  # (the blocks that take a second piece are few when the pieces are few more than the blocks)
            by_length = max(1.0, sum(pieces) * nkv / slots) * (largest + setup)
        return by_request, by_length * keys

    def decode_by_length(self, ctx_lens, nkv: int, hd: int | None = None) -> bool:
        """Whether a decode step over contexts of these lengths should use the kernel that deals
        key tiles by length (:meth:`_dealt_estimates`)."""
        if self.decode_balanced in ("0", "1"):
            return self.decode_balanced == "1"
        by_request, by_length = self._dealt_estimates(ctx_lens, nkv, hd)
        return by_request > by_length

    def prefill_key_split(self, blocks: int, hd: int, max_ctx_len: int) -> int:
        """Among how many blocks the tcgen05 prefill kernel shares the keys of a query tile: the
        count that costs least by this estimate, in key tiles one block walks: rounds of blocks over
        the device, each block its share of the longest context's key tiles plus a start and end
        worth six, and for the block that adds the shares three key tiles and 1.1 per share
        (measured, a 128-token portion at 2,048 tokens, us for 1 / 2 / 4 / 8 shares: 23.9 / 18.5 / 17.0 /
        19.0; at 8,192 tokens: 81 / 47.6 / 36.8 / 29.5; a 512-token portion at 8,192: 103 / 65 / 72 / 82);
        if that saves a quarter of the time and leaves every block four key tiles; 1 when the tiles
        fill the device anyway."""
        slots = self.sm_count * (2 if hd == 64 else 1)
        if blocks <= 0 or blocks >= slots:
            return 1
        key_tiles = max(max_ctx_len // 64, 1)

        def cost(ks: int) -> float:
            rounds = -(-blocks * ks // slots)
            return rounds * (key_tiles / ks + 6.0) + (3.0 + 1.1 * ks if ks > 1 else 0.0)

        limit = max(1, min(16, max_ctx_len // 256))
        least = min(cost(ks) for ks in range(1, limit + 1))
        best = next(ks for ks in range(1, limit + 1) if cost(ks) <= 1.05 * least)  # (the fewest shares among the near-best)
        return best if cost(best) <= 0.75 * cost(1) else 1

    def paged_attention(self, q, k_cache, v_cache, block_tables, ctx, nh, nkv, hd, page_size,
                        scale, window, out, ragged: bool | None = None) -> None:
        """Attention of every token of the step over its request's cached keys and values.
        bfloat16 with a head size the tensor-core kernels take and at most 16 query heads per
        key/value head: requests with few rows go to the split decode kernel, longer portions
        to the prefill kernel.  Everything else (32-bit, other head sizes) runs the general
        kernel, whose order of operations does not depend on the batch."""
        if hd % 8 or hd > 256:
            raise KernelError(f"head_dim {hd} is not supported: it must be a multiple of 8, at most 256")
        if nkv < 1 or nh % nkv:
            raise KernelError(f"{nh} query heads cannot share {nkv} key/value heads")
        groups = nh // nkv
        if q.dtype == self.torch.bfloat16 and hd in ATTENTION_HEAD_DIMS and groups <= 16:
            lib = self._attention_lib(hd)
            # which requests go to which kernel: the same for every layer of the step
            # (kept on the step's context, one per (heads per key/value head, head size): mixers
            # of different shapes in one model each get their own)
            plans = getattr(ctx, "_attention_plans", None)
            if plans is None:
                plans = ctx._attention_plans = {}
            plan = plans.get((groups, hd))
            bounds = getattr(ctx, "bounds", None)
            if plan is None and bounds is not None:
                # a launch of fixed size (a captured step): both kernels, over as many query tiles
                # as any step within the bounds can have; each kernel skips the other's requests
                tokens, seqs, max_ctx = bounds
                rows = lib.ie_attention_prefill_rows()
                tiles = seqs + tokens // rows
                # (the keys of a tile may be shared among blocks here too: how many is decided from the
                # bounds alone, for the tiles a step of so many tokens usually has: one request's portion
                # and little else; blocks for tiles that a step does not have leave at once)
                likely = tokens // rows + min(seqs, 2)
                plan = plans[(groups, hd)] = {"any": True, "all": False, "tiles": tiles, "tile_pairs": tiles,
                                              "max_ctx": max_ctx, "likely_tiles": likely}
            if plan is None:
                small = [ql * groups <= 16 for ql in ctx.q_lens]
                plan = {"small": small, "any": any(small), "all": all(small)}
                if not plan["all"]:
                    rows = lib.ie_attention_prefill_rows()
                    per_seq = [-(-ql // rows) for ql, s in zip(ctx.q_lens, small) if not s]
                    plan["tiles"] = sum(per_seq)
                    plan["tile_pairs"] = sum(-(-t // 2) for t in per_seq)
                plans[(groups, hd)] = plan
            args = (q, k_cache, v_cache, block_tables, ctx, nh, nkv, hd, page_size, scale, window, out)
            if plan["any"]:
                if ragged is None:
                    ragged = max(getattr(ctx, "ragged", ()) or (0,))
                self._decode_attention(lib, int(ragged) if bounds is None else self.BY_REQUEST, *args)
            if not plan["all"]:
                self._prefill_attention(lib, plan, *args)
            return
        self.paged_attention_general(q, k_cache, v_cache, block_tables, ctx, nh, nkv, hd, page_size,
                                     scale, window, out)

    def _scratch(self, ctx, name: str, floats: int, device):
        ws = getattr(ctx, "ws", None)
        if ws is not None:
            # (one row of exactly what is asked for, rounded up so that it seldom has to grow: the
            # workspace's own floor of rows is for per-token buffers)
            size = max(1 << max(int(floats) - 1, 0).bit_length(), 1 << 22)  # (16 MB at least: most steps never outgrow it)
            return ws.buffer(name, 1, size, self.torch.float32, rows_cap=None)[:, :floats]
        return self.torch.empty(floats, dtype=self.torch.float32, device=device)

    @_kind("attention.decode")
    def _decode_attention(self, lib, ragged, q, k_cache, v_cache, block_tables, ctx, nh, nkv, hd, page_size, scale,
                          window, out) -> None:
        """The requests with few rows (the kernels skip the others): key tiles dealt by length
        when the step's context says its lengths differ much, else by request."""
        total_pages, stream = k_cache.shape[0], self._stream()
        by_length = self.decode_balanced == "1" or (self.decode_balanced == "auto" and ragged == self.BY_LENGTH)
        if by_length and ctx.num_seqs <= lib.ie_attention_decode_balanced_max_seqs():
            per_pair = self.decode_balanced_blocks_per_pair
            floats = lib.ie_attention_decode_balanced_scratch_floats(ctx.num_seqs, nkv, per_pair)
            scratch = self._scratch(ctx, "attn.partial", floats, q.device)
            tickets = self._decode_tickets(ctx.num_seqs * nkv)
            self._check(lib.ie_attention_decode_balanced(
                q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_tables.data_ptr(),
                block_tables.shape[1], ctx.cu_q.data_ptr(), ctx.ctx_lens.data_ptr(), out.data_ptr(),
                scratch.data_ptr(), tickets.data_ptr(), ctx.num_seqs, nh, nkv, page_size,
                total_pages, scale, window, per_pair, self._err_ptr, stream), "attention_decode_balanced")
            self.balanced_launches += 1
            return
        splits = self.decode_splits(ctx.num_seqs, nkv, block_tables.shape[1] * page_size, hd)
        floats = lib.ie_attention_decode_scratch_floats(ctx.num_seqs, nkv, splits)
        scratch = tickets = None
        if floats:
            scratch = self._scratch(ctx, "attn.partial", floats, q.device)
            tickets = self._decode_tickets(ctx.num_seqs * nkv)
        self._check(lib.ie_attention_decode_ordered(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_tables.data_ptr(),
            block_tables.shape[1], ctx.cu_q.data_ptr(), ctx.ctx_lens.data_ptr(), out.data_ptr(),
            self._ptr(scratch), self._ptr(tickets), ctx.num_seqs, nh, nkv, page_size,
            total_pages, scale, window, splits, self._ptr(getattr(ctx, "decode_order", None)),
            ragged if ragged in (self.SMALL_2, self.SMALL_3) and splits == 1 else 0, self._err_ptr, stream),
            "attention_decode")

    @_kind("attention.prefill")
    def _prefill_attention(self, lib, plan, q, k_cache, v_cache, block_tables, ctx, nh, nkv, hd, page_size,
                           scale, window, out) -> None:
        """The requests with more than 16 rows, in query tiles of `ie_attention_prefill_rows` tokens."""
        total_pages, stream = k_cache.shape[0], self._stream()
        tiles = plan["tiles"]
        fixed = "max_ctx" in plan  # a launch of fixed size: nothing is decided from the step's own lengths
        max_ctx = plan["max_ctx"] if fixed else ctx.max_ctx_len
        if self.attn_tc5 and lib.ie_attention_prefill_tc5_ok(page_size, max_ctx):
            # Head sizes 64 and 128, pages of 8 tokens or more: the tcgen05 / TMEM / TMA kernel.
            # While the blocks would fill the GPU less than about twice, a block takes two tiles
            # of a request, a late (long) and an early (short) one.  With so few tiles that even
            # then much of the GPU would idle (a short portion of a long prompt), the keys of
            # every tile are shared among several blocks instead.
            ksplit = 1
            if self.prefill_key_splits:
                ksplit = self.prefill_key_split((plan["likely_tiles"] if fixed else tiles) * nh, hd, max_ctx)
            # (pairs of tiles only where single tiles would take more than one round of blocks: two
            # prompts of 256 tokens took 11.2 us in pairs, 8.3 in single tiles; eight of them 14.9 and 17.5)
            slots = self.sm_count * (2 if hd == 64 else 1)
            paired = (not fixed and ksplit == 1 and slots < tiles * nh <= self.prefill_paired_max * self.sm_count)
            # (portions at the end of long contexts: their tiles see about as many keys each, and pairs
            # would only halve the blocks where those do not fill the device anyway: two 512-token
            # portions at 65,536 tokens took 1,602 us in 128 blocks of two tiles, 826 in 256 of one)
            if paired and ctx.max_ctx_len >= 2 * max(ctx.q_lens) and plan["tile_pairs"] * nh < slots:
                paired = False
            if paired:
                tiles = plan["tile_pairs"]
            scratch = tickets = None
            if ksplit > 1:
                floats = lib.ie_attention_prefill_tc5_scratch_floats(tiles, nh, ksplit)
                scratch = self._scratch(ctx, "attn.prefill_partial", floats, q.device)
                tickets = self._decode_tickets(max(tiles * nh, ctx.num_seqs * nkv))
            self._check(lib.ie_attention_prefill_tc5(
                q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_tables.data_ptr(),
                block_tables.shape[1], ctx.cu_q.data_ptr(), ctx.ctx_lens.data_ptr(), out.data_ptr(),
                ctx.num_tokens, ctx.num_seqs, tiles, 1 if paired else 0, nh, nkv, page_size, total_pages,
                scale, window, ksplit, self._ptr(scratch), self._ptr(tickets), self._err_ptr, stream),
                "attention_prefill_tc5")
            return
        self._check(lib.ie_attention_prefill(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_tables.data_ptr(),
            block_tables.shape[1], ctx.cu_q.data_ptr(), ctx.ctx_lens.data_ptr(), out.data_ptr(),
            ctx.num_seqs, tiles, nh, nkv, page_size, total_pages, scale, window,
            self._err_ptr, stream), "attention_prefill")

    @_kind("attention.general")
    def paged_attention_general(self, q, k_cache, v_cache, block_tables, ctx, nh, nkv, hd,
                                page_size, scale, window, out) -> None:
        self._check(self._paged_attention_generic(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), _dtype_code(q),
            block_tables.data_ptr(), block_tables.shape[1], ctx.seq_of_token.data_ptr(),
            ctx.positions.data_ptr(), out.data_ptr(), ctx.num_tokens, nh, nkv, hd, page_size,
            k_cache.shape[0], scale, window, self._err_ptr, self._stream()), "paged_attention")

    @_kind("activation")
    def silu_mul(self, gate_up, out, interleave: int = 0) -> None:
        """``out[n, i] = silu(gate_i) * up_i`` from rows that hold the gates and then the ups
        (``interleave`` 0) or gates and ups alternating in blocks of ``interleave`` values."""
        parts, stride = self._partials(gate_up)
        self._check(self._silu_mul(gate_up.data_ptr(), _dtype_code(gate_up), parts, stride,
                                   out.data_ptr(), _dtype_code(out), out.shape[0], out.shape[1],
                                   interleave, self._stream()), "silu_mul")

    GATE_BLOCK = 16  # rows of gates, then of ups, alternate in blocks of this many in a fused matrix

    def gated_linear(self, x, w_gate_up, interleave: int, *, ws, tag="ffn", out_dtype=None):
        """``silu(x @ gate^T) * (x @ up^T)`` with gate and up stacked in ``w_gate_up`` (halves, or
        alternating in blocks of ``interleave`` rows).  A step of few rows whose matrix is laid
        out in blocks of ``GATE_BLOCK`` runs one kernel that streams the weights and applies the
        activation to the sums it holds; everything else is the product followed by
        :meth:`silu_mul`."""
        torch = self.torch
        m, k = x.shape
        n = w_gate_up.shape[0]
        act = ws.buffer(tag + ".act", m, n // 2, out_dtype or x.dtype)
        tiles = -(-n // 128)
        if (self.gated_gemm and interleave == self.GATE_BLOCK and x.dtype == torch.bfloat16
                and act.dtype == torch.bfloat16 and 0 < m <= self.FEW_ROWS and self.few_row_gemm == "tma"
                and k % 8 == 0 and k <= 2048 and n % 32 == 0 and x.is_contiguous() and w_gate_up.is_contiguous()
                and tiles <= (self.tma_max_tiles if m <= 8 else self.tma_max_tiles_wide)
                and tiles <= self.tma_max_blocks):
            self._gated(x, w_gate_up, act)
            return act
        gate_up = self.linear(x, w_gate_up, ws=ws, tag=tag + ".gate_up", out_dtype=act.dtype, allow_split=True)
        self.silu_mul(gate_up, act, interleave)
        return act

    @_kind("linear:ffn.gate_up")
    def _gated(self, x, w, act) -> None:
        self._check(self._gemm_tma_gated_bf16(x.data_ptr(), w.data_ptr(), act.data_ptr(), x.shape[0], w.shape[0],
                                              x.shape[1], self._err_ptr, self._stream()), "gemm_tma_gated")

    def argmax(self, logits, out) -> None:
        """Greedy token of every row (lowest index on ties)."""
        rows = logits.shape[0]
        chunks = max(1, min(2 * self.sm_count // max(rows, 1), 64))
        need = 2 * rows * chunks
        if self._argmax_scratch is None or self._argmax_scratch.numel() < need:
            self._argmax_scratch = self.torch.empty(max(need, 4096), dtype=self.torch.int32, device=self.device)
        self._check(self._argmax(logits.data_ptr(), rows, logits.shape[1], chunks,
                                 self._argmax_scratch.data_ptr(), out.data_ptr(), self._stream()), "argmax")
        self.launches += 1

    @_kind("sampling")
    def sample(self, logits, out, temperature=None, top_k=None, top_p=None, min_p=None,
               penalty=None, seen_bits=None, seeds=None, draws=None, logprob=None) -> None:
        """One token per row of 32-bit ``logits``; the per-row tensors are optional (absent:
        greedy, no cut-off, no penalty).  ``seeds`` and ``draws`` (int64) are needed as soon
        as ``temperature`` is given."""
        if temperature is None and penalty is None and logprob is None:
            return self.argmax(logits, out)
        self._check(self._sample(
            logits.data_ptr(), logits.shape[0], logits.shape[1], self._ptr(temperature),
            self._ptr(top_k), self._ptr(top_p), self._ptr(min_p), self._ptr(penalty),
            self._ptr(seen_bits), 0 if seen_bits is None else seen_bits.shape[1],
            self._ptr(seeds), self._ptr(draws), out.data_ptr(), self._ptr(logprob),
            self._stream()), "sample")


_OPS: dict[str, CudaOps] = {}


def get_ops(device="cuda") -> CudaOps:
    """The process-wide kernel set for ``device``; built and loaded on first use."""
    key = str(device)
    if key not in _OPS:
        _OPS[key] = CudaOps(device)
    return _OPS[key]
