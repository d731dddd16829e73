"""The scheduler's decisions: budget, portions, admission order, what happens when pages run
out, finishing and freeing (engine/runtime/scheduler.py of the reference is the model)."""

from __future__ import annotations

import pytest

from inference_engine_b200.cache import CacheManager, PagedGroupSpec
from inference_engine_b200.engine.scheduler import Scheduler, SeqStatus, Sequence
from inference_engine_b200.sampling.params import SamplingParams


def _sched(num_pages=16, page_size=4, max_num_seqs=4, budget=16, chunked=True):
    cache = CacheManager([PagedGroupSpec(1, 1, 8, None)], [], num_pages, page_size, max_num_seqs)
    return Scheduler(cache, max_num_seqs, budget, chunked), cache


def _seq(i, prompt_len, max_tokens=8):
    return Sequence(i, f"r{i}", list(range(prompt_len)), SamplingParams(max_tokens=max_tokens))


def _run(sched, batch, sample=True):
    """What the engine does after a step: count the tokens, append a sampled one."""
    for seq, n in zip(batch.seqs, batch.num_tokens):
        seq.num_computed += n
        if sample and seq.num_computed == seq.length:
            seq.output_ids.append(0)


def test_budget_must_cover_one_token_per_running_request():
    with pytest.raises(ValueError, match="max_num_batched_tokens"):
        _sched(max_num_seqs=8, budget=4)


def test_prompts_are_cut_into_portions_under_the_budget():
    sched, cache = _sched(budget=10)
    a, b = _seq(0, 25), _seq(1, 3)
    sched.add(a)
    sched.add(b)
    batch = sched.schedule()
    assert (batch.seqs, batch.num_tokens) == ([a], [10])  # the head takes the whole budget
    _run(sched, batch)
    batch = sched.schedule()
    assert batch.num_tokens == [10] and batch.total_tokens == 10
    _run(sched, batch)
    batch = sched.schedule()  # 5 left for a, then b is admitted with what remains
    assert (batch.seqs, batch.num_tokens) == ([a, b], [5, 3])
    _run(sched, batch)
    batch = sched.schedule()  # both decode: one token each, running requests first
    assert (batch.seqs, batch.num_tokens) == ([a, b], [1, 1])
    assert a.status == b.status == SeqStatus.RUNNING


def test_without_chunked_prefill_a_prompt_runs_whole_or_waits():
    sched, _ = _sched(budget=10, chunked=False, num_pages=32)
    a, b, c = _seq(0, 6), _seq(1, 7), _seq(2, 14)
    for s in (a, b, c):
        sched.add(s)
    batch = sched.schedule()
    assert (batch.seqs, batch.num_tokens) == ([a], [6])  # b does not fit the 4 that are left
    _run(sched, batch)
    batch = sched.schedule()
    assert (batch.seqs, batch.num_tokens) == ([a, b], [1, 7])
    _run(sched, batch)
    sched.finish(a, "length")
    sched.finish(b, "length")
    batch = sched.schedule()  # larger than the whole budget: runs alone with all of it
    assert (batch.seqs, batch.num_tokens) == ([c], [14])


def test_admission_is_first_come_first_served_and_never_skips_the_head():
    sched, cache = _sched(num_pages=4, page_size=4, budget=64)
    big, small = _seq(0, 14, max_tokens=2), _seq(1, 2, max_tokens=2)
    blocker = _seq(2, 9, max_tokens=2)
    sched.add(blocker)
    _run(sched, sched.schedule())  # blocker holds 3 of 4 pages
    sched.add(big)
    sched.add(small)
    batch = sched.schedule()
    assert batch.seqs == [blocker]  # big cannot start; small must not overtake it
    assert list(sched.waiting) == [big, small] and not cache.has_request(big.seq_id)
    sched.finish(blocker, "stop")
    batch = sched.schedule()
    assert batch.seqs[0] is big


def test_max_num_seqs_limits_admission():
    sched, _ = _sched(max_num_seqs=2, budget=32)
    seqs = [_seq(i, 3) for i in range(3)]
    for s in seqs:
        sched.add(s)
    batch = sched.schedule()
    assert batch.seqs == seqs[:2] and list(sched.waiting) == [seqs[2]]
    _run(sched, batch)
    sched.finish(seqs[0], "stop")
    assert sched.schedule().seqs == [seqs[1], seqs[2]]


def test_when_pages_run_out_the_newest_running_request_is_preempted():
    sched, cache = _sched(num_pages=6, page_size=4, budget=32)
    old, mid, new = _seq(0, 8, 16), _seq(1, 8, 16), _seq(2, 7, 16)
    for s in (old, mid, new):
        sched.add(s)
    _run(sched, sched.schedule())  # 2 + 2 + 2 pages: the pool is full
    assert cache.num_free_pages == [0]
    batch = sched.schedule()  # old and mid need a new page each; new (7 -> 8) still fits its own
    # old asks first: the newest not yet scheduled (new) is preempted and gives back 2 pages
    assert batch.seqs == [old, mid] and new.status == SeqStatus.WAITING
    assert new.num_computed == 0 and new.num_preemptions == 1 and sched.num_preemptions == 1
    assert list(sched.waiting) == [new] and not cache.has_request(new.seq_id)
    assert len(new.output_ids) == 1  # what it produced is kept and prefilled again later
    _run(sched, batch)
    cache.check_invariants()


def test_a_request_preempts_itself_when_nobody_newer_is_left():
    sched, cache = _sched(num_pages=4, page_size=4, max_num_seqs=2, budget=16)
    a, b = _seq(0, 8, max_tokens=4), _seq(1, 4, max_tokens=4)
    sched.add(a)
    sched.add(b)
    _run(sched, sched.schedule())  # a holds 2 pages, b 1; one is free
    batch = sched.schedule()  # a takes the last page; b needs one too and nobody newer is left
    assert batch.seqs == [a] and b.status == SeqStatus.WAITING and b.num_preemptions == 1
    assert list(sched.waiting) == [b] and not cache.has_request(b.seq_id)
    assert cache.num_free_pages == [1]  # b's page came back, but b now needs two: it waits
    cache.check_invariants()


def test_preempted_requests_return_oldest_first_and_prefill_their_outputs_again():
    sched, cache = _sched(num_pages=6, page_size=4, budget=64)
    a, b, c = _seq(0, 8, 16), _seq(1, 8, 16), _seq(2, 8, 16)
    for s in (a, b, c):
        sched.add(s)
    _run(sched, sched.schedule())
    batch = sched.schedule()
    assert batch.seqs == [a, b] and list(sched.waiting) == [c]  # c (newest) went first
    _run(sched, batch)
    for _ in range(3):  # fill a's and b's third pages
        _run(sched, sched.schedule())
    batch = sched.schedule()  # a needs a fourth page: b (newest running) is preempted
    assert batch.seqs == [a] and list(sched.waiting) == [b, c]  # the older victim is in front
    _run(sched, batch)
    sched.finish(a, "length")
    batch = sched.schedule()
    assert batch.seqs[0] is b and batch.num_tokens[0] == b.length  # prompt + produced tokens, in one go
    assert b.num_computed == 0 and b.length == 8 + len(b.output_ids)


def test_requests_that_can_never_fit_are_refused_and_finish_frees_at_once():
    sched, cache = _sched(num_pages=4, page_size=4)
    with pytest.raises(ValueError, match="exceeds the KV cache"):
        sched.add(_seq(0, 10, max_tokens=7))
    a = _seq(1, 10, max_tokens=6)
    sched.add(a)
    _run(sched, sched.schedule())
    assert cache.num_free_pages == [1]
    sched.finish(a, "stop")
    assert cache.num_free_pages == [4] and a.status == SeqStatus.FINISHED and a.finish_reason == "stop"
    assert not sched.has_unfinished() and sched.schedule() is None


def test_abort_from_either_queue():
    sched, cache = _sched()
    a, b = _seq(0, 5), _seq(1, 5)
    sched.add(a)
    _run(sched, sched.schedule())
    sched.add(b)
    assert sched.abort("r1") is b and sched.abort("r0") is a and sched.abort("r0") is None
    assert a.finish_reason == "abort" and cache.num_free_pages == [16]
