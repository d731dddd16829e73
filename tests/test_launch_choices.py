"""The host-side choices among kernel launches (no GPU needed: they are arithmetic on lengths).

`CudaOps.decode_by_length` picks between the two decode attention launches from the step's context
lengths, `CudaOps.prefill_key_split` among how many blocks the prefill attention shares a query
tile's keys, `CudaOps.decode_splits` into how many parts the by-request decode attention cuts a
context.
"""

from __future__ import annotations

import types

from inference_engine_b200.kernels.cuda_ops import CudaOps


def _ops(sm_count=148, balanced="auto", split_target=128, cluster_max=8):
    ops = types.SimpleNamespace(sm_count=sm_count, decode_balanced=balanced, decode_split_target=split_target,
                                decode_cluster_max=cluster_max, decode_cluster_tokens=4096)
    ops.decode_splits = lambda num_seqs, nkv, table_tokens=0, hd=None: CudaOps.decode_splits(ops, num_seqs, nkv, table_tokens, hd)
    ops._dealt_estimates = lambda lens, nkv, hd=None: CudaOps._dealt_estimates(ops, lens, nkv, hd)
    return ops


def test_contexts_are_cut_only_for_small_batches():
    ops = _ops()
    # 2, 4 or 8 parts merge inside a thread-block cluster: counts are rounded down to one of those
    assert CudaOps.decode_splits(ops, 1, 8) == 8
    assert CudaOps.decode_splits(ops, 3, 8) == 4   # (5 would fit the target)
    assert CudaOps.decode_splits(ops, 8, 8) == 2
    assert CudaOps.decode_splits(ops, 16, 8) == 1
    assert CudaOps.decode_splits(ops, 64, 8) == 1
    # ... except when the tables hold long contexts: as many parts as give nearly every SM a block
    assert CudaOps.decode_splits(ops, 1, 8, table_tokens=8192) == 16
    assert CudaOps.decode_splits(ops, 1, 8, table_tokens=2048) == 8
    assert CudaOps.decode_splits(ops, 1, 1, table_tokens=32768) == 32  # never more than 32 parts
    assert CudaOps.decode_splits(ops, 2, 8, table_tokens=8192) == 9    # 144 blocks
    assert CudaOps.decode_splits(ops, 3, 8, table_tokens=8192) == 6
    assert CudaOps.decode_splits(ops, 5, 8, table_tokens=8192) == 3    # (the cluster sizes would leave it at 2)
    assert CudaOps.decode_splits(ops, 8, 8, table_tokens=8192) == 2
    assert CudaOps.decode_splits(ops, 32, 8, table_tokens=8192) == 1
    assert CudaOps.decode_splits(ops, 12, 8, table_tokens=8192) == 3   # 288 half-size blocks on 296 slots, not 96 on 148
    assert CudaOps.decode_splits(ops, 16, 8, table_tokens=8192) == 1   # (128 blocks either way)
    plain = _ops(cluster_max=0)
    assert CudaOps.decode_splits(plain, 1, 8) == 16 and CudaOps.decode_splits(plain, 3, 8) == 5
    # all clusters of a launch have to run at one time: where the device fits fewer clusters of 8
    # than there are (request, head) pairs, the parts are clusters of 4
    ops._clusters_at_once = lambda hd, parts: {8: 14, 4: 33, 2: 70}[parts]
    assert CudaOps.decode_splits(ops, 1, 8, hd=64) == 8      # 8 clusters of 8
    assert CudaOps.decode_splits(ops, 2, 8, hd=64) == 4      # 16 clusters of 8 would take two rounds
    assert CudaOps.decode_splits(ops, 2, 8) == 8             # (without a head size nothing is asked)
    assert CudaOps.decode_splits(ops, 7, 2, hd=64) == 8      # 14 pairs
    assert CudaOps.decode_splits(ops, 4, 8, hd=64) == 4
    ops._clusters_at_once = lambda hd, parts: 0              # unknown: as before
    assert CudaOps.decode_splits(ops, 2, 8, hd=64) == 8


def test_work_is_dealt_by_length_only_where_that_pays():
    ops = _ops()
    by_length = lambda lens, nkv=8: CudaOps.decode_by_length(ops, lens, nkv)
    assert by_length([32768] + [256] * 31)          # one long context among short ones
    assert by_length([8000] + [500] * 7)
    assert by_length([4352, 128] * 16)              # half long, half short, more pairs than SMs
    assert not by_length([1024] * 8)                # equal lengths: the by-request launch is a trip to memory shorter
    assert not by_length([2304] * 32)
    assert not by_length([100, 2000, 700, 1500, 300, 900, 1200, 400])  # small differences do not pay for the set-up
    assert not by_length([64 + 31 * i for i in range(64)])  # 512 pairs: the hardware's dispatch evens them out
    # more pairs than block slots and lengths that differ by a factor: the hardware's dispatch fills the gaps
    assert not by_length([128 + (1920 * ((7 * i) % 40)) // 39 for i in range(40)])
    # equal lengths, a few blocks more than the device runs at once: a second round for those few
    assert by_length([4096] * 40)
    assert not by_length([4096] * 36)               # 288 blocks on 296 slots
    assert not by_length([1024] * 48) and not by_length([1024] * 64)
    # up to one pair per SM: that kernel's blocks start again for every stretch of another pair
    assert not by_length([4096] * 12) and not by_length([2048] * 11)
    assert by_length([32768] * 7) and by_length([8192] * 10) and by_length([32768, 256, 256, 256])
    assert not by_length([8192] * 16) and not by_length([4096] * 18)
    assert by_length([4096] * 9)   # 72 pairs on 148 SMs: two pieces per pair, all at once
    # the switch overrides the estimate
    assert CudaOps.decode_by_length(_ops(balanced="1"), [1024] * 8, 8)
    assert not CudaOps.decode_by_length(_ops(balanced="0"), [32768] + [256] * 31, 8)


def test_keys_of_a_query_tile_are_shared_when_tiles_are_few_and_contexts_long():
    ops = _ops()
    split = lambda blocks, hd, ctx: CudaOps.prefill_key_split(ops, blocks, hd, ctx)
    assert split(128, 64, 4096) == 2      # 4 tiles x 32 heads on 296 block slots
    assert split(96, 128, 4096) == 1      # head size 128: one block per SM, 148 slots; three shares would take two rounds
    assert split(32, 64, 2048) == 4 and split(32, 64, 8192) == 8   # one tile: 17.0 us (23.9 unshared), 29.5 (81)
    assert split(128, 64, 512) == 1       # a whole 512-token prompt: few keys per tile (11.1 us; 19.0 in two shares)
    assert split(512, 64, 4096) == 1      # the tiles fill the device
    assert split(200, 64, 4000) == 1      # two thirds full: sharing would not save a quarter
    assert split(128, 64, 200) == 1       # too short a context to share
    for blocks in (1, 8, 32, 64, 128):
        for ctx in (256, 1024, 8192, 131072):
            ks = split(blocks, 64, ctx)
            assert 1 <= ks <= 16 and ks <= max(1, ctx // 256)


def test_the_history_masks_of_the_repetition_penalty_grow_with_the_histories():
    """The sampler keeps every request's bit mask from step to step (by the request's key) and adds
    only the ids that are new; the result is the mask built from the whole history."""
    import numpy as np
    import torch

    from inference_engine_b200.sampling.params import SamplingParams
    from inference_engine_b200.sampling.sampler import Sampler

    vocab = 1000
    sampler = Sampler(ops=None, device="cpu", vocab_size=vocab)
    rng = np.random.default_rng(0)
    params = [SamplingParams(temperature=0.7, repetition_penalty=1.2), SamplingParams(temperature=0.7),
              SamplingParams(temperature=0.7, repetition_penalty=1.1)]
    histories = [list(rng.integers(0, vocab, 40)), list(rng.integers(0, vocab, 5)), list(rng.integers(0, vocab, 300))]

    def expected(hists):
        bits = np.zeros((len(hists), (vocab + 31) // 32), dtype=np.uint32)
        for r, (p, h) in enumerate(zip(params, hists)):
            if p.repetition_penalty != 1.0:
                for t in h:
                    bits[r, t >> 5] |= np.uint32(1) << np.uint32(t & 31)
        return bits

    for step in range(6):
        got = sampler._seen_bits(params, histories, keys=["a", "b", "c"]).numpy().view(np.uint32)
        assert (got == expected(histories)).all()
        histories = [h + [int(rng.integers(0, vocab))] for h in histories]
    # another request under a known key (a shorter history): its mask starts again
    histories[0] = [3, 4]
    got = sampler._seen_bits(params, histories, keys=["a", "b", "c"]).numpy().view(np.uint32)
    assert (got == expected(histories)).all()
    # without keys every mask is built from the whole history
    got = sampler._seen_bits(params, histories).numpy().view(np.uint32)
    assert (got == expected(histories)).all()


def test_many_requests_of_one_length_run_in_small_blocks():
    """`CudaOps.decode_dealing`: by request in blocks of 3 or 2 warps when the step's (request, head)
    pairs then need fewer rounds over the device and no context is so much longer than the others
    that its block would be the last by far; by length or in the larger blocks otherwise."""
    ops = _ops()
    fits = {(64, 4): 2, (64, 3): 3, (64, 2): 4, (128, 4): 1, (128, 3): 1, (128, 2): 2}
    ops.decode_small, ops._force_small, ops._decode_blocks_per_sm = True, 0, lambda hd, warps: fits[(hd, warps)]
    ops.decode_by_length = lambda lens, nkv, hd=None: CudaOps.decode_by_length(ops, lens, nkv, hd)
    ops._clusters_at_once = lambda hd, parts: 0
    ops._by_request_estimate = CudaOps._by_request_estimate
    for name in ("BY_REQUEST", "BY_LENGTH", "SMALL_2", "SMALL_3"):
        setattr(ops, name, getattr(CudaOps, name))
    ops._dealing_look, ops._dealing_answer = None, 0
    ops._decode_dealing = lambda lens, nkv, hd=None: CudaOps._decode_dealing(ops, lens, nkv, hd)
    deal = lambda lens, nkv=8, hd=64: CudaOps.decode_dealing(ops, lens, nkv, hd)
    assert deal([1024] * 40) == CudaOps.SMALL_3 and deal([1024] * 55) == CudaOps.SMALL_3  # up to 444 blocks: one round
    assert deal([1024] * 56) == CudaOps.SMALL_2 and deal([1024] * 74) == CudaOps.SMALL_2  # up to 592
    assert deal([1024] * 80) == CudaOps.SMALL_3     # two rounds of three-warp blocks against three of four-warp ones
    assert deal([1024] * 128) == CudaOps.SMALL_2    # two rounds against four
    assert deal([1024] * 160) == CudaOps.SMALL_3    # three against five
    assert deal([800 + 8 * i for i in range(48)]) == CudaOps.SMALL_3    # (lengths that differ a little)
    assert deal([1024] * 37) == CudaOps.BY_REQUEST       # 296 blocks: one round of the larger ones
    assert deal([1024] * 64, hd=None) == CudaOps.BY_REQUEST
    import random
    rng = random.Random(0)
    assert deal([rng.randint(64, 2048) for _ in range(64)]) == CudaOps.BY_REQUEST
    assert deal([rng.randint(128, 2048) for _ in range(40)]) == CudaOps.BY_REQUEST
    assert deal([rng.randint(512, 1536) for _ in range(48)]) == CudaOps.BY_REQUEST
    assert deal([rng.randint(768, 1280) for _ in range(40)]) == CudaOps.SMALL_3
    assert deal([256] * 39 + [32768]) == CudaOps.BY_LENGTH
    # long contexts, more pairs than SMs but fewer than block slots: the blocks' shares by length are more even
    assert deal([8192] * 24) == CudaOps.BY_LENGTH and deal([4096] * 24) == CudaOps.BY_LENGTH
    assert deal([8192] * 32) == CudaOps.BY_REQUEST and deal([4096] * 28) == CudaOps.BY_REQUEST and deal([2048] * 24) == CudaOps.BY_REQUEST
    assert deal([4096] * 48) == CudaOps.SMALL_3   # (by length would beat the four-warp blocks' two rounds, not these)
    # the estimate itself: whole rounds for one length; else every later request starts as one of the round before ends
    est = CudaOps._by_request_estimate
    assert est([1000] * 80, 37, 1.0, 300.0) == 3 * 1300
    assert est([900, 800, 700, 100, 50], 3, 1.0, 0.0) == max(700 + 100, 800 + 50, 900)
    # the answer is kept while the batch looks the same (every context a token longer: the same look)
    calls = []
    ops._decode_dealing = lambda lens, nkv, hd=None: calls.append(1) or CudaOps._decode_dealing(ops, lens, nkv, hd)
    assert deal([1030] * 40) == deal([1031] * 40) == deal([1032] * 40) == CudaOps.SMALL_3 and len(calls) == 1
    assert deal([1030] * 41) == CudaOps.SMALL_3 and len(calls) == 2
    ops.decode_small = False
    assert deal([1024] * 64) == CudaOps.BY_REQUEST


def test_scratch_buffers_are_sized_as_asked():
    """The attention kernels' scratch is one row of what they ask for (rounded up, 16 MB at least), not
    the workspace's floor of rows for per-token buffers; a larger request grows it once."""
    import torch

    from inference_engine_b200.engine.workspace import Workspace

    ops = types.SimpleNamespace(torch=torch)
    ctx = types.SimpleNamespace(ws=Workspace("cpu", min_rows=4096))
    small = CudaOps._scratch(ops, ctx, "attn.partial", 1000, "cpu")
    assert tuple(small.shape) == (1, 1000) and ctx.ws.bytes() == 4 << 22
    version = ctx.ws.version
    again = CudaOps._scratch(ops, ctx, "attn.partial", 3_000_000, "cpu")
    assert tuple(again.shape) == (1, 3_000_000) and ctx.ws.version == version and again.data_ptr() == small.data_ptr()
    large = CudaOps._scratch(ops, ctx, "attn.partial", 5_000_000, "cpu")
    assert tuple(large.shape) == (1, 5_000_000) and ctx.ws.version == version + 1 and ctx.ws.bytes() == 4 << 23
