"""The engine's loop on the host: a runner and a sampler of the test's own stand in for the
device (the next token is a function of the tokens so far), the scheduler and the cache manager
are the real ones.  Covered: a step that fails when it is launched, a step that turns out to
have failed when its tokens are read, and an end-of-sequence token that arrives for a sequence
which was preempted while that token was still on its way.

The reference's counterpart: TestServingEngineStepFailureRecovery
(internal/engine/serving_test.go:327) with a runner whose Step returns an error; its engine
fails the step's sequences and frees what they held (internal/engine/serving.go:199-202, 646-666)."""
import hashlib
from types import SimpleNamespace

import pytest

from gollmgo_b200.cache import CacheManager, PagedKVNeed
from gollmgo_b200.config import EngineConfig
from gollmgo_b200.engine.llm_engine import Engine
from gollmgo_b200.engine.sequence import SeqState
from gollmgo_b200.sampling import SamplingParams

EOS = 7


def fake_token(tokens):
    return int.from_bytes(hashlib.sha256(repr(list(tokens)).encode()).digest()[:2], "little") % 900 + 10


class StubRunner:
    """step(entries) keeps the cache manager's books the way the real runner does (all or
    nothing) and "computes" the next token of every wanted place from the request's history."""

    def __init__(self, num_pages, page, max_requests=16, next_token=fake_token):
        self.spec = SimpleNamespace(vocab_size=1000, eos_token_ids=(EOS,))
        self.cache = CacheManager([PagedKVNeed(1, 8, None)], page, num_pages, max_requests=max_requests)
        self.max_model_len = 10_000
        self.device = "cpu"
        self.last_tokens = None
        self.history = {}
        self.prev = []                     # tokens "on the device": what the last step sampled, by row
        self.calls = 0
        self.fail_step_at = set()          # calls of step() that raise
        self.fail_check_at = set()         # calls of check_kernels() that raise
        self.checks = 0
        self.next_token = next_token

    def step(self, entries):
        self.calls += 1
        if self.calls in self.fail_step_at:
            raise RuntimeError("simulated GPU error")
        admitted, starts = [], {}
        try:
            for e in entries:
                if e.request_id not in self.cache.requests:
                    self.cache.admit(e.request_id)
                    admitted.append(e.request_id)
                    self.history[e.request_id] = []
                starts[e.request_id] = self.cache.num_tokens(e.request_id)
            for e in entries:
                self.cache.append(e.request_id, len(e.tokens))
        except Exception:
            for rid, n in starts.items():
                if self.cache.num_tokens(rid) > n:
                    self.cache.rollback(rid, n)
            for rid in admitted:
                self.cache.free(rid)
            raise
        out = []
        for e in entries:
            h = self.history[e.request_id]
            assert len(h) == starts[e.request_id], "the engine fed a position twice or skipped one"
            toks = [self.prev[e.token_src]] if e.token_src >= 0 else list(e.tokens)
            h.extend(toks)
            for w in e.want:
                assert w == len(toks) - 1
                out.append(self.next_token(h))
        return out

    def check_kernels(self, wait=True):
        self.checks += 1
        if self.checks in self.fail_check_at:
            raise RuntimeError("a kernel gave up on a bounded wait")


class StubSampler:
    def __init__(self, runner):
        self.runner = runner

    def sample_async(self, logits, params, draw_index):
        self.runner.prev = list(logits)
        return list(logits)

    def wait(self, handle):
        return handle


def make_engine(num_pages=64, page=4, next_token=fake_token, **cfg):
    runner = StubRunner(num_pages, page, next_token=next_token)
    ecfg = EngineConfig(block_size=page, num_blocks=num_pages, cuda_graphs=False, **cfg)
    return Engine(runner=runner, sampler=StubSampler(runner), engine_config=ecfg), runner


def plain_generate(prompt, n, next_token=fake_token, eos=True):
    toks, out = list(prompt), []
    for _ in range(n):
        t = next_token(toks)
        out.append(t)
        toks.append(t)
        if eos and t == EOS:
            break
    return out


PROMPTS = [[1, 2, 3, 4, 5], [9, 8], [4] * 11, [6, 6, 6], [3, 1, 4, 1, 5, 9, 2, 6]]


def drain(eng):
    results = []
    guard = 0
    while eng.has_unfinished():
        results.extend(eng.step())
        guard += 1
        assert guard < 10_000
    return results


def test_undisturbed_run_equals_plain_generation():
    eng, runner = make_engine(max_batch_size=3, max_token_budget=16, prefill_chunk_size=4)
    outs = eng.generate(PROMPTS, SamplingParams(max_tokens=9))
    assert [o.token_ids for o in outs] == [plain_generate(p, 9) for p in PROMPTS]
    runner.cache.audit()
    assert runner.cache.free_pages() == 64 and not runner.cache.requests


@pytest.mark.parametrize("fail_at", [1, 2, 3, 5, 8])
def test_a_step_that_fails_at_launch_ends_its_sequences_and_the_queue_goes_on(fail_at):
    eng, runner = make_engine(max_batch_size=2, max_token_budget=16, prefill_chunk_size=4)
    runner.fail_step_at = {fail_at}
    rids = [eng.enqueue(p, SamplingParams(max_tokens=9)) for p in PROMPTS]
    results = drain(eng)
    failed = [r for r in results if r.error]
    assert failed and all(r.finished and r.finish_reason == "error" and r.token_id == -1 for r in failed)
    assert "simulated GPU error" in failed[0].error
    assert len(failed) <= 2 and eng.stats.failed_steps == 1 and eng.stats.failed_requests == len(failed)
    bad = {r.request_id for r in failed}
    for rid, p in zip(rids, PROMPTS):
        o = eng.output_of(rid)
        want = plain_generate(p, 9)
        if rid in bad:
            # what it had produced before the failure is kept and is right; nothing after it
            assert o.finish_reason == "error" and o.error and o.token_ids == want[:len(o.token_ids)]
            assert len(o.token_ids) < len(want)
        else:
            assert o.token_ids == want and o.finish_reason in ("length", "stop")
    # every request got exactly one last result
    last = [r for r in results if r.finished]
    assert sorted(r.request_id for r in last) == sorted(rids)
    runner.cache.audit()
    assert runner.cache.free_pages() == 64 and not runner.cache.requests
    assert runner.cache.slots.num_free == runner.cache.slots.max_requests
    # and the engine is as good as new
    again = eng.generate([PROMPTS[0]], SamplingParams(max_tokens=9))[0]
    assert again.token_ids == plain_generate(PROMPTS[0], 9)


@pytest.mark.parametrize("fail_at", [1, 2, 4, 7])
def test_a_step_found_failed_when_its_tokens_are_read_voids_the_step_launched_since(fail_at):
    """check_kernels() raises when the tokens of step n are read, one turn after step n+1 was
    launched: the sequences of both end with an error, the rest of the queue is served."""
    eng, runner = make_engine(max_batch_size=2, max_token_budget=16, prefill_chunk_size=4)
    runner.fail_check_at = {fail_at}
    rids = [eng.enqueue(p, SamplingParams(max_tokens=9)) for p in PROMPTS]
    results = drain(eng)
    failed = {r.request_id for r in results if r.error}
    assert failed and eng.stats.failed_steps == 1
    served = 0
    for rid, p in zip(rids, PROMPTS):
        o = eng.output_of(rid)
        want = plain_generate(p, 9)
        if rid in failed:
            assert o.finish_reason == "error" and o.token_ids == want[:len(o.token_ids)]
            assert -1 not in o.token_ids
        else:
            assert o.token_ids == want
            served += 1
    assert served >= 1
    assert sorted(r.request_id for r in results if r.finished) == sorted(rids)
    runner.cache.audit()
    assert runner.cache.free_pages() == 64 and not runner.cache.requests


def test_out_of_pages_inside_the_step_is_a_failed_step_not_a_crash():
    """A cache that refuses what the scheduler planned (here: pages taken behind the
    scheduler's back) fails the step's sequences; nothing is left half-appended."""
    eng, runner = make_engine(num_pages=8, page=4, max_batch_size=2, max_token_budget=32, prefill_chunk_size=0)
    rid = eng.enqueue([5] * 10, SamplingParams(max_tokens=4))
    runner.cache.admit("thief")
    real_schedule = eng.scheduler.schedule

    def schedule_then_steal():
        out = real_schedule()
        runner.cache.append("thief", 4 * runner.cache.free_pages())       # every page that is left
        return out
    eng.scheduler.schedule = schedule_then_steal
    results = eng.step()
    assert [r.finish_reason for r in results] == ["error"] and "OutOfPages" in results[0].error
    assert eng.output_of(rid).finish_reason == "error"
    runner.cache.free("thief")
    runner.cache.audit()
    assert runner.cache.free_pages() == 8 and not eng.has_unfinished()


def test_end_token_that_arrives_after_its_sequence_was_preempted():
    """Turn k+1 preempts a decoding sequence whose token of step k is still on the device; the
    token then turns out to be the end-of-sequence token.  The sequence ends where it is (in
    the queue, holding nothing) instead of raising WAITING -> FINISHED.  Swept over the place of
    the end token so that the case is certainly met; every output equals plain generation."""
    hit = 0
    for eos_at in range(1, 26):
        def next_token(tokens, eos_at=eos_at):
            # request "b" (prompt of 4 sixes) ends with its eos_at-th generated token
            if tokens[:4] == [6, 6, 6, 6] and len(tokens) == 4 + eos_at - 1:
                return EOS
            return fake_token(tokens)
        eng, runner = make_engine(num_pages=12, page=4, next_token=next_token, max_batch_size=4,
                                  max_token_budget=32, prefill_chunk_size=0)
        seen = []
        real_finish = eng.scheduler.finish

        def finish(seq, reason, seen=seen, real_finish=real_finish):
            seen.append((seq.request_id, seq.state, reason))
            real_finish(seq, reason)
        eng.scheduler.finish = finish
        a = eng.enqueue([1, 2, 3, 4, 5, 6, 7], SamplingParams(max_tokens=30), request_id="a")
        b = eng.enqueue([6, 6, 6, 6], SamplingParams(max_tokens=30), request_id="b")
        drain(eng)
        oa, ob = eng.output_of(a), eng.output_of(b)
        assert oa.token_ids == plain_generate([1, 2, 3, 4, 5, 6, 7], 30, next_token)
        assert ob.token_ids == plain_generate([6, 6, 6, 6], 30, next_token)
        assert ob.finish_reason == "stop" and ob.token_ids[-1] == EOS and len(ob.token_ids) == eos_at
        assert eng.sequences[b].state is SeqState.FINISHED
        assert all(s is not eng.sequences[b] for s in eng.scheduler.waiting)
        hit += any(rid == "b" and state is SeqState.WAITING and reason == "stop" for rid, state, reason in seen)
        runner.cache.audit()
        assert runner.cache.free_pages() == 12 and not runner.cache.requests
    assert hit >= 1, "the sweep never preempted the sequence while its end token was on its way"


def test_generate_as_a_closed_loop_keeps_no_more_requests_in_the_engine_than_asked():
    """concurrency = 3 (the reference's serving benchmark drives its server this way): never more
    than three requests are admitted or waiting, every prompt is served, in the order given,
    with the tokens it gets alone; a failed request makes room like a finished one."""
    eng, runner = make_engine(num_pages=64)
    runner.fail_step_at = {9}
    seen = []
    step = eng.step

    def counted():
        seen.append(len(eng.scheduler.running) + len(eng.scheduler.waiting))
        return step()
    eng.step = counted
    prompts = [[20 + i, 3, 5 + i % 4] * (1 + i % 3) for i in range(11)]
    outs = eng.generate(prompts, SamplingParams(max_tokens=6), concurrency=3)
    assert max(seen) == 3 and len(outs) == len(prompts)
    failed = [o for o in outs if o.finish_reason == "error"]
    assert 1 <= len(failed) <= 3
    for p, o in zip(prompts, outs):
        assert o.prompt_token_ids == p
        if o.finish_reason != "error":
            assert o.token_ids == plain_generate(p, 6)
    runner.cache.audit()
    assert not runner.cache.requests
    with pytest.raises(ValueError, match="concurrency"):
        eng.generate(prompts[:1], SamplingParams(max_tokens=2), concurrency=-1)
