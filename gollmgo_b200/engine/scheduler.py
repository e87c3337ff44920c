"""First-come-first-served continuous batching with chunked prefill.

Each ``schedule()`` plans one step under ``max_batch_size`` sequences and
``max_token_budget`` tokens, in the reference's order
(internal/scheduler/fcfs.go:72-164): first every decoding sequence, one token
each; then sequences in the middle of their prompt, a portion each
(``prefill_chunk_size`` at most, cut to the budget that is left, down to one
token); then new requests in arrival order.

Where this differs from the reference, on purpose:
  * the plan says how many tokens each sequence gets, and the engine runs exactly
    that (the reference's engine recomputes the portion and may exceed the
    budget: internal/engine/serving.go:353-362);
  * free pages are consulted.  A new request is admitted only if its first
    portion fits beside one more page for every running sequence, and the head
    of the queue blocks those behind it (strict arrival order);
  * when pages run out for the running sequences, the one admitted last is
    preempted: its pages are given back, it returns to the front of the queue
    and is later recomputed over prompt and generated tokens as one prompt, so
    the tokens it goes on to generate are the same.  (The reference preempts the
    sequence with most blocks at 95 % utilisation and, on re-admission, does not
    rebuild the keys and values of generated tokens: internal/engine/serving.go:717-798,
    364-373.)
  * a request that could never fit (prompt + max_tokens beyond the pool or the
    longest sequence allowed) is refused when it is added.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional

from ..config import EngineConfig
from .sequence import SeqState, Sequence


class QueueFull(RuntimeError):
    pass


class RequestTooLong(ValueError):
    pass


@dataclass
class Scheduled:
    seq: Sequence
    num_tokens: int

    @property
    def samples(self) -> bool:
        """True if this portion reaches the sequence's last known token, so that
        its last logits give the next token."""
        return self.seq.num_computed + self.num_tokens == self.seq.total_len


@dataclass
class SchedulerOutput:
    scheduled: List[Scheduled] = field(default_factory=list)
    preempted: List[Sequence] = field(default_factory=list)
    decode_tokens: int = 0
    prefill_tokens: int = 0


class Scheduler:
    def __init__(self, cfg: EngineConfig, cache, max_model_len: int):
        self.cfg = cfg
        self.cache = cache
        self.max_model_len = max_model_len
        self.waiting: Deque[Sequence] = deque()
        self.running: Dict[int, Sequence] = {}        # admitted: prefilling or decoding
        self.admit_order: List[int] = []              # ids in the order of (re-)admission
        self.num_preemptions = 0

    # ------------------------------------------------------------------ queue
    def capacity_tokens(self) -> int:
        """Most tokens one request may hold: the model's longest sequence, and what the
        cache manager says a single request can ever keep (it knows which groups slide)."""
        portion = min(self.cfg.prefill_chunk_size or self.cfg.max_token_budget, self.cfg.max_token_budget)
        cap = self.cache.capacity_tokens(portion)
        return self.max_model_len if cap is None else min(self.max_model_len, cap)

    def add(self, seq: Sequence) -> None:
        if self.cfg.max_queue_depth > 0 and len(self.waiting) >= self.cfg.max_queue_depth:
            raise QueueFull(f"queue is full: depth {len(self.waiting)}")
        need = len(seq.prompt) + seq.params.max_tokens
        limit = self.capacity_tokens()
        if not seq.prompt:
            raise RequestTooLong("a request needs at least one prompt token")
        if need > limit:
            raise RequestTooLong(f"request needs {need} tokens (prompt {len(seq.prompt)} + "
                                 f"max_tokens {seq.params.max_tokens}); at most {limit} fit")
        self.waiting.append(seq)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ pages
    def _preempt(self, seq: Sequence, out: SchedulerOutput) -> None:
        seq.transition(SeqState.PREEMPTED)
        seq.num_computed = 0
        seq.preemptions += 1
        self.num_preemptions += 1
        del self.running[seq.id]
        self.admit_order.remove(seq.id)
        if seq.id in self.cache.requests:
            self.cache.free(seq.id)
        seq.transition(SeqState.WAITING)
        self.waiting.appendleft(seq)
        out.preempted.append(seq)

    # ------------------------------------------------------------------ one step's plan
    def schedule(self) -> SchedulerOutput:
        out = SchedulerOutput()
        cfg = self.cfg
        budget = cfg.max_token_budget
        chunk_cap = cfg.prefill_chunk_size or (1 << 30)
        # Free pages per cache group as this plan uses them up.  What a portion takes and what a
        # sliding group gives back first is asked of the cache manager (pages_delta), in the order
        # in which the step will append, so a plan that is accepted here is one the cache accepts.
        free: List[int] = self.cache.free_pages_per_group()
        page, sliding = self.cache.page_size, self.cache.any_window
        planned: List[Scheduled] = []
        deltas: Dict[int, list] = {}                     # seq id -> its (taken, given back) per group
        planned_new: List[Sequence] = []                # admitted in this step (each takes a state slot)

        def fits(delta) -> bool:
            return all(take <= f + back for (take, back), f in zip(delta, free))

        def book(delta, sign: int) -> None:
            for g, (take, back) in enumerate(delta):
                free[g] -= sign * (take - back)

        def fits_or_preempt(seq: Sequence, n: int) -> bool:
            """Make room for n tokens of seq by preempting later-admitted sequences
            (never an earlier one).  False if seq itself had to go."""
            if n == 1 and not sliding and seq.num_computed % page:
                return True                              # lands in a page the sequence holds: nothing to ask or book
            delta = self.cache.pages_delta(seq.id, n)
            while not fits(delta):
                victim_id = self.admit_order[-1]
                victim = self.running[victim_id]
                # a victim already planned in this step loses its plan
                for i, s in enumerate(planned):
                    if s.seq is victim:
                        booked = deltas.pop(victim.id, None)
                        if booked is not None:
                            book(booked, -1)
                        planned.pop(i)
                        break
                held = self.cache.pages_held(victim.id)
                self._preempt(victim, out)
                for g, h in enumerate(held):
                    free[g] += h
                if victim is seq:
                    return False
            book(delta, +1)
            deltas[seq.id] = delta
            return True

        # 1. decoding sequences, oldest first, one token each
        for sid in sorted(self.running):
            seq = self.running.get(sid)
            if seq is None or seq.state is not SeqState.DECODING:
                continue
            if len(planned) >= cfg.max_batch_size or budget <= 0:
                break
            if fits_or_preempt(seq, 1):
                planned.append(Scheduled(seq, 1))
                budget -= 1
        # 2. sequences in the middle of their prompt
        for sid in sorted(self.running):
            seq = self.running.get(sid)
            if seq is None or seq.state is not SeqState.PREFILLING:
                continue
            if len(planned) >= cfg.max_batch_size or budget <= 0:
                break
            n = min(seq.remaining, chunk_cap, budget)
            if n > 0 and fits_or_preempt(seq, n):
                planned.append(Scheduled(seq, n))
                budget -= n
        # 3. new requests in arrival order; one that does not fit blocks the rest (strict_fcfs)
        #    or is passed over
        skipped: List[Sequence] = []
        while self.waiting and len(planned) < cfg.max_batch_size and budget > 0:
            seq = self.waiting[0]
            if any(seq is p for p in out.preempted):
                break                                   # just preempted: not in the same step
            n = min(seq.remaining, chunk_cap, budget)
            delta = self.cache.pages_delta(None, n)
            reserve = len(self.running)                 # one more page for everyone who is running
            room = all(take + reserve <= f for (take, _), f in zip(delta, free))
            if not room or self.cache.slots.num_free <= len(planned_new):
                if cfg.strict_fcfs:
                    break
                skipped.append(self.waiting.popleft())
                continue
            self.waiting.popleft()
            seq.transition(SeqState.PREFILLING)
            self.running[seq.id] = seq
            self.admit_order.append(seq.id)
            planned_new.append(seq)
            book(delta, +1)
            deltas[seq.id] = delta
            planned.append(Scheduled(seq, n))
            budget -= n
        for seq in reversed(skipped):
            self.waiting.appendleft(seq)
        for s in planned:
            if s.seq.state is SeqState.DECODING:
                out.decode_tokens += s.num_tokens
            else:
                out.prefill_tokens += s.num_tokens
        out.scheduled = planned
        return out

    # ------------------------------------------------------------------ after the step
    def advance(self, s: Scheduled) -> None:
        """The step ran: s.num_tokens more tokens of the sequence are cached."""
        seq = s.seq
        seq.num_computed += s.num_tokens
        if seq.state is SeqState.PREFILLING and seq.num_computed < seq.total_len:
            seq.transition(SeqState.PREFILLING)

    def token_sampled(self, seq: Sequence) -> None:
        if seq.state is SeqState.PREFILLING:
            seq.transition(SeqState.DECODING)

    def finish(self, seq: Sequence, reason: str) -> None:
        """End a sequence wherever it is: running, or back in the queue after a preemption
        (its last token, still on the device when it was preempted, may be the one that ends
        it; its pages are gone already).  Finishing twice only changes the reason."""
        seq.finish_reason = reason
        if seq.state is SeqState.FINISHED:
            return
        if seq.state in (SeqState.WAITING, SeqState.PREEMPTED):
            self.waiting = deque(s for s in self.waiting if s is not seq)
            seq.state = SeqState.WAITING
        seq.transition(SeqState.FINISHED)
        self.running.pop(seq.id, None)
        if seq.id in self.admit_order:
            self.admit_order.remove(seq.id)
        if seq.id in self.cache.requests:
            self.cache.free(seq.id)
