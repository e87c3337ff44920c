"""The scheduler's decisions, on the host, with the real cache manager and a fake
model whose next token is a function of the tokens so far."""
import hashlib

import pytest

from gollmgo_b200.cache import CacheManager, PagedKVNeed
from gollmgo_b200.config import EngineConfig
from gollmgo_b200.engine import (QueueFull, RequestTooLong, Scheduler, SeqState, Sequence)
from gollmgo_b200.sampling import SamplingParams


def make(num_pages=64, page=4, **cfg):
    ecfg = EngineConfig(block_size=page, num_blocks=num_pages, **cfg)
    cache = CacheManager([PagedKVNeed(1, 8, None)], page, num_pages, max_requests=16)
    return Scheduler(ecfg, cache, max_model_len=10_000), cache


def seq(i, n_prompt, max_tokens=4):
    return Sequence(i, f"r{i}", list(range(1, n_prompt + 1)), SamplingParams(max_tokens=max_tokens))


def fake_token(tokens):
    return int.from_bytes(hashlib.sha256(repr(tokens).encode()).digest()[:2], "little") % 1000 + 10


def run_step(sched, cache):
    """What the engine does with a plan: reserve cache room, advance, sample, finish."""
    out = sched.schedule()
    for s in out.scheduled:
        if s.seq.id not in cache.requests:
            cache.admit(s.seq.id)
        cache.append(s.seq.id, s.num_tokens)
    for s in out.scheduled:
        samples = s.samples
        sched.advance(s)
        if samples:
            s.seq.output.append(fake_token(s.seq.tokens))
            sched.token_sampled(s.seq)
            if len(s.seq.output) >= s.seq.params.max_tokens:
                sched.finish(s.seq, "length")
    cache.audit()
    return out


def drain(sched, cache, limit=10_000):
    steps = 0
    while sched.has_work():
        out = run_step(sched, cache)
        assert out.scheduled or out.preempted, "no progress"
        steps += 1
        assert steps < limit
    return steps


def test_admission_in_arrival_order_and_first_token():
    sched, cache = make(prefill_chunk_size=0)
    a, b = seq(0, 5), seq(1, 3)
    sched.add(a), sched.add(b)
    out = run_step(sched, cache)
    assert [(s.seq.id, s.num_tokens) for s in out.scheduled] == [(0, 5), (1, 3)]
    assert a.state is SeqState.DECODING and len(a.output) == 1 and a.num_computed == 5
    out = run_step(sched, cache)
    assert [(s.seq.id, s.num_tokens) for s in out.scheduled] == [(0, 1), (1, 1)]
    assert out.decode_tokens == 2 and out.prefill_tokens == 0


def test_decode_first_then_running_prompts_then_new_requests():
    sched, cache = make(prefill_chunk_size=4, max_token_budget=100)
    sched.add(seq(0, 2))
    run_step(sched, cache)                       # 0 is decoding now
    sched.add(seq(1, 10))
    run_step(sched, cache)                       # 1 took its first portion
    sched.add(seq(2, 3))
    out = run_step(sched, cache)
    assert [(s.seq.id, s.num_tokens) for s in out.scheduled] == [(0, 1), (1, 4), (2, 3)]
    assert out.decode_tokens == 1 and out.prefill_tokens == 7


def test_prompt_is_cut_into_portions_across_steps():
    sched, cache = make(prefill_chunk_size=4)
    a = seq(0, 10)
    sched.add(a)
    sizes = []
    while a.state is not SeqState.DECODING:
        out = run_step(sched, cache)
        sizes.append(out.scheduled[0].num_tokens)
        assert (len(a.output) == 1) == (a.num_computed == 10)
    assert sizes == [4, 4, 2]


def test_token_budget_cuts_the_portion_and_is_never_exceeded():
    sched, cache = make(prefill_chunk_size=0, max_token_budget=8)
    sched.add(seq(0, 2, max_tokens=50))
    run_step(sched, cache)
    sched.add(seq(1, 20))
    sched.add(seq(2, 5))
    out = run_step(sched, cache)
    assert [(s.seq.id, s.num_tokens) for s in out.scheduled] == [(0, 1), (1, 7)]     # 1 + 7 = budget
    for _ in range(6):
        out = run_step(sched, cache)
        assert sum(s.num_tokens for s in out.scheduled) <= 8
        assert out.scheduled[0].seq.id == 0      # decoding is never starved by prompts


def test_batch_size_cap():
    sched, cache = make(max_batch_size=2, prefill_chunk_size=0)
    for i in range(4):
        sched.add(seq(i, 2, max_tokens=2))
    out = run_step(sched, cache)
    assert [s.seq.id for s in out.scheduled] == [0, 1]
    out = run_step(sched, cache)                 # both finish here (2 tokens each)
    assert [s.seq.id for s in out.scheduled] == [0, 1]
    out = run_step(sched, cache)
    assert [s.seq.id for s in out.scheduled] == [2, 3]


def test_queue_depth_and_requests_that_can_never_fit():
    sched, cache = make(num_pages=8, page=4, max_queue_depth=2)
    sched.add(seq(0, 2)), sched.add(seq(1, 2))
    with pytest.raises(QueueFull):
        sched.add(seq(2, 2))
    sched2, _ = make(num_pages=8, page=4)
    with pytest.raises(RequestTooLong):
        sched2.add(seq(0, 30, max_tokens=4))     # 34 tokens, the pool holds 32
    with pytest.raises(RequestTooLong):
        sched2.add(Sequence(1, "e", [], SamplingParams()))
    sched2.add(seq(2, 28, max_tokens=4))


def test_head_of_queue_blocks_those_behind_it():
    sched, cache = make(num_pages=6, page=4, prefill_chunk_size=0)
    sched.add(seq(0, 12, max_tokens=3))          # 3 pages, then a 4th while decoding
    run_step(sched, cache)
    sched.add(seq(1, 12, max_tokens=2))          # needs 3 pages + 1 in reserve: does not fit (3 free)
    sched.add(seq(2, 2, max_tokens=2))           # would fit, but must wait its turn
    out = run_step(sched, cache)
    assert [s.seq.id for s in out.scheduled] == [0]
    assert [s.id for s in sched.waiting] == [1, 2]
    drain(sched, cache)
    assert cache.free_pages() == 6


def test_when_pages_run_out_the_last_admitted_is_preempted_and_recomputed():
    sched, cache = make(num_pages=4, page=4, prefill_chunk_size=0)
    a, b = seq(0, 7, max_tokens=8), seq(1, 4, max_tokens=8)
    sched.add(a), sched.add(b)
    run_step(sched, cache)                       # a: 2 pages, b: 1 page
    assert a.state is b.state is SeqState.DECODING
    preempted_at = None
    for step in range(40):
        out = run_step(sched, cache)
        if out.preempted:
            preempted_at = step
            assert [s.id for s in out.preempted] == [1]          # the later one goes, never the earlier
            assert b.state is SeqState.WAITING and b.num_computed == 0 and sched.waiting[0] is b
            assert 1 not in cache.requests
            break
    assert preempted_at is not None
    kept = list(b.output)
    drain(sched, cache)
    assert a.finished and b.finished and b.preemptions >= 1
    assert b.output[:len(kept)] == kept and len(b.output) == 8
    assert cache.free_pages() == 4


def test_results_do_not_depend_on_pool_size_or_portions():
    def run(num_pages, chunk, budget):
        sched, cache = make(num_pages=num_pages, page=4, prefill_chunk_size=chunk, max_token_budget=budget)
        seqs = [seq(i, n, max_tokens=m) for i, (n, m) in enumerate([(9, 6), (1, 9), (17, 3), (5, 12), (30, 2)])]
        for s in seqs:
            sched.add(s)
        drain(sched, cache)
        assert all(g.pool.num_free == num_pages for g in cache.groups) and cache.slots.num_free == 16
        return [s.output for s in seqs], sched.num_preemptions
    roomy, p0 = run(200, 0, 4096)
    tight, p1 = run(10, 3, 7)
    assert roomy == tight and p0 == 0 and p1 > 0


def test_state_machine_refuses_wrong_transitions():
    from gollmgo_b200.engine import InvalidTransition
    s = seq(0, 3)
    with pytest.raises(InvalidTransition):
        s.transition(SeqState.DECODING)
    s.transition(SeqState.PREFILLING)
    s.transition(SeqState.DECODING)
    s.transition(SeqState.FINISHED)
    with pytest.raises(InvalidTransition):
        s.transition(SeqState.WAITING)


def test_without_strict_fcfs_a_request_that_does_not_fit_is_passed_over():
    sched, cache = make(num_pages=6, page=4, prefill_chunk_size=0, strict_fcfs=False)
    sched.add(seq(0, 12, max_tokens=3))
    run_step(sched, cache)
    sched.add(seq(1, 12, max_tokens=2))          # does not fit beside request 0
    sched.add(seq(2, 2, max_tokens=2))           # fits: goes ahead of request 1
    out = run_step(sched, cache)
    assert [s.seq.id for s in out.scheduled] == [0, 2]
    assert [s.id for s in sched.waiting] == [1]
    drain(sched, cache)
    assert cache.free_pages() == 6


def make_groups(needs, num_pages, page, **cfg):
    ecfg = EngineConfig(block_size=page, num_blocks=num_pages, **cfg)
    cache = CacheManager(needs, page, num_pages, max_requests=16)
    return Scheduler(ecfg, cache, max_model_len=10_000), cache


def test_a_group_with_a_window_is_planned_by_what_the_cache_manager_says():
    """Every layer slides (window 8, pages of 4 tokens, 7 pages): a request far longer than the
    pool fits, because pages behind the window go back as it grows; the plan never asks the
    cache for more than it can give (run_step would raise OutOfPages), and two requests share
    the small pool by preemption where they must."""
    sched, cache = make_groups([PagedKVNeed(1, 8, 8)], 7, 4, prefill_chunk_size=4, max_token_budget=8)
    a, b = seq(0, 30, max_tokens=40), seq(1, 9, max_tokens=25)
    sched.add(a), sched.add(b)                   # 70 and 34 tokens in a pool of 28
    drain(sched, cache)
    assert a.finished and b.finished and len(a.output) == 40 and len(b.output) == 25
    assert cache.free_pages() == 7 and not cache.requests
    # the same outputs as on a pool where nothing is ever short
    sched2, cache2 = make_groups([PagedKVNeed(1, 8, 8)], 200, 4, prefill_chunk_size=4, max_token_budget=8)
    a2, b2 = seq(0, 30, max_tokens=40), seq(1, 9, max_tokens=25)
    sched2.add(a2), sched2.add(b2)
    drain(sched2, cache2)
    assert (a.output, b.output) == (a2.output, b2.output) and sched2.num_preemptions == 0


def test_the_group_that_keeps_every_key_sets_the_limit_beside_one_that_slides():
    needs = [PagedKVNeed(1, 8, 8), PagedKVNeed(1, 8, None)]
    sched, cache = make_groups(needs, 10, 4, prefill_chunk_size=4, max_token_budget=8)
    assert len(cache.groups) == 2 and sched.capacity_tokens() == 40
    with pytest.raises(RequestTooLong):
        sched.add(seq(0, 30, max_tokens=11))
    seqs = [seq(1, 20, max_tokens=20), seq(2, 7, max_tokens=12), seq(3, 15, max_tokens=9)]
    for s in seqs:
        sched.add(s)
    drain(sched, cache)
    assert all(s.finished for s in seqs) and sched.num_preemptions > 0
    assert [g.pool.num_free for g in cache.groups] == [10, 10]


def test_a_model_without_pages_is_never_short_of_them():
    from gollmgo_b200.cache import FixedStateNeed
    sched, cache = make_groups([FixedStateNeed((4,))], 1, 4, prefill_chunk_size=4, max_token_budget=8)
    assert not cache.groups and sched.capacity_tokens() == 10_000
    seqs = [seq(i, 50 + i, max_tokens=30) for i in range(3)]
    for s in seqs:
        sched.add(s)
    drain(sched, cache)
    assert all(s.finished for s in seqs) and sched.num_preemptions == 0


def test_finishing_a_sequence_that_waits_again_after_a_preemption():
    sched, cache = make(num_pages=4, page=4, prefill_chunk_size=0)
    a, b = seq(0, 7, max_tokens=8), seq(1, 4, max_tokens=8)
    sched.add(a), sched.add(b)
    for _ in range(40):
        out = run_step(sched, cache)
        if out.preempted:
            break
    assert b.state is SeqState.WAITING and sched.waiting[0] is b
    sched.finish(b, "stop")
    assert b.finished and b.finish_reason == "stop" and not sched.waiting
    sched.finish(b, "abort")                     # twice: only the reason changes
    assert b.finished and b.finish_reason == "abort"
    drain(sched, cache)
    assert a.finished and cache.free_pages() == 4
