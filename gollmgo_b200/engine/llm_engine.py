"""The engine: requests in, tokens out.  One loop ticks the scheduler, builds the
step's batch, runs the step function, samples, and finishes sequences.

Shape of the loop and of the public calls follows the reference's ServingEngine
(internal/engine/serving.go:160-204 loop, 308-461 runStep, 465-490 emit,
670-691 Enqueue, 800-823 cleanup) and its Request{ID, TokenIDs, MaxTokens}
(internal/engine/engine.go:7-11); it runs in the caller's thread instead of a
goroutine: ``step()`` is one turn of the loop, ``generate()`` runs it to the end.
"""
from __future__ import annotations

import random
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence as Seq

import torch

from ..config import EngineConfig, read_config_json
from ..sampling.params import SamplingParams
from .batch import StepEntry
from .runner import ModelRunner
from .scheduler import Scheduler, SchedulerOutput
from .sequence import SeqState, Sequence


@dataclass
class TokenResult:
    """One generated token (the reference's TokenResult: internal/engine/engine.go:14-20)."""
    request_id: str
    token_id: int
    finished: bool
    finish_reason: Optional[str] = None


@dataclass
class RequestOutput:
    request_id: str
    prompt_token_ids: List[int]
    token_ids: List[int]
    finish_reason: Optional[str]
    ttft_s: Optional[float] = None
    e2e_s: Optional[float] = None
    token_times: List[float] = field(default_factory=list)
    preemptions: int = 0


@dataclass
class EngineStats:
    steps: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    generated_tokens: int = 0
    preemptions: int = 0
    pages_high_water: int = 0


class Engine:
    def __init__(self, model: Optional[str] = None, *, config: Optional[dict] = None,
                 weights_seed: Optional[int] = None, engine_config: Optional[EngineConfig] = None,
                 **engine_options):
        """``model``: a folder with config.json and *.safetensors.  Or ``config`` (a
        config.json dict) with ``weights_seed`` for random weights made on the device.
        Engine options (EngineConfig fields) may be given as keywords."""
        ecfg = engine_config or EngineConfig(**engine_options)
        if model is not None:
            self.runner = ModelRunner(read_config_json(model), ecfg, weights=model)
        elif config is not None:
            self.runner = ModelRunner(config, ecfg, weights_seed=weights_seed if weights_seed is not None else 0)
        else:
            raise ValueError("give a model folder, or a config with weights_seed")
        from ..sampling.sampler import Sampler
        self.ecfg = ecfg
        self.spec = self.runner.spec
        self.scheduler = Scheduler(ecfg, self.runner.cache, self.runner.max_model_len)
        self.sampler = Sampler(self.runner.device, max(ecfg.max_batch_size, 1))
        self.sequences: Dict[str, Sequence] = {}
        self.stats = EngineStats()
        self._next_id = 0
        self._seed_rng = random.Random()
        self._stopped = False

    # ------------------------------------------------------------------ requests
    def enqueue(self, token_ids: Seq[int], params: Optional[SamplingParams] = None,
                request_id: Optional[str] = None, **param_options) -> str:
        """Add a request; returns its id.  ``params`` or SamplingParams fields as keywords
        (max_tokens, temperature, top_k, top_p, seed, ignore_eos)."""
        if self._stopped:
            raise RuntimeError("engine is stopped")
        params = params or SamplingParams(**param_options)
        params.validate()
        if params.seed is None and not params.greedy:
            params = SamplingParams(**{**params.__dict__, "seed": self._seed_rng.getrandbits(63)})
        V = self.spec.vocab_size
        for t in token_ids:
            if not (0 <= int(t) < V):
                raise ValueError(f"token id {t} is outside [0, {V})")
        seq_id = self._next_id
        self._next_id += 1
        rid = request_id if request_id is not None else f"req-{seq_id}"
        if rid in self.sequences and not self.sequences[rid].finished:
            raise ValueError(f"request id {rid!r} is in use")
        seq = Sequence(seq_id, rid, [int(t) for t in token_ids], params)
        self.scheduler.add(seq)
        self.sequences[rid] = seq
        return rid

    def has_unfinished(self) -> bool:
        return self.scheduler.has_work()

    # ------------------------------------------------------------------ one turn of the loop
    def step(self) -> List[TokenResult]:
        plan: SchedulerOutput = self.scheduler.schedule()
        self.stats.preemptions += len(plan.preempted)
        if not plan.scheduled:
            if self.scheduler.has_work() and not plan.preempted:
                raise RuntimeError("scheduler made no progress: the page pool is too small for the "
                                   "request at the head of the queue")
            return []
        entries, samplers = [], []
        for s in plan.scheduled:
            seq = s.seq
            toks = seq.token_slice(seq.num_computed, seq.num_computed + s.num_tokens)
            entries.append(StepEntry(seq.id, toks, [s.num_tokens - 1] if s.samples else []))
            if s.samples:
                samplers.append(seq)
        logits = self.runner.step(entries)
        tokens = self.sampler.sample(logits, [q.params for q in samplers], [len(q.output) for q in samplers]) \
            if samplers else []
        self.runner.check_kernels()
        now = time.perf_counter()
        for s in plan.scheduled:
            self.scheduler.advance(s)
        results = []
        eos = set(self.spec.eos_token_ids)
        for seq, tok in zip(samplers, tokens):
            seq.output.append(int(tok))
            seq.token_times.append(now)
            if seq.first_token_at is None:
                seq.first_token_at = now
            seq.last_token_at = now
            self.scheduler.token_sampled(seq)
            reason = None
            if not seq.params.ignore_eos and tok in eos:
                reason = "stop"
            elif len(seq.output) >= seq.params.max_tokens:
                reason = "length"
            if reason:
                self.scheduler.finish(seq, reason)
            results.append(TokenResult(seq.request_id, int(tok), reason is not None, reason))
        st = self.stats
        st.steps += 1
        st.prefill_tokens += plan.prefill_tokens
        st.decode_tokens += plan.decode_tokens
        st.generated_tokens += len(tokens)
        st.pages_high_water = max(g.pool.high_water for g in self.runner.cache.groups)
        return results

    # ------------------------------------------------------------------ whole requests
    def generate(self, prompts: Seq[Seq[int]], params=None, **param_options) -> List[RequestOutput]:
        """Generate for every prompt (token ids); returns outputs in the order given.
        ``params``: one SamplingParams for all, or one per prompt."""
        if params is None:
            params = SamplingParams(**param_options)
        plist = list(params) if isinstance(params, (list, tuple)) else [params] * len(prompts)
        if len(plist) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        rids = []
        pending = list(zip(prompts, plist))
        i = 0
        while i < len(pending) or self.has_unfinished():
            while i < len(pending) and (self.ecfg.max_queue_depth <= 0
                                        or len(self.scheduler.waiting) < self.ecfg.max_queue_depth):
                rids.append(self.enqueue(pending[i][0], pending[i][1]))
                i += 1
            self.step()
        return [self.output_of(r) for r in rids]

    def output_of(self, request_id: str) -> RequestOutput:
        seq = self.sequences[request_id]
        return RequestOutput(seq.request_id, list(seq.prompt), list(seq.output), seq.finish_reason,
                             (seq.first_token_at - seq.created_at) if seq.first_token_at else None,
                             (seq.last_token_at - seq.created_at) if seq.last_token_at else None,
                             list(seq.token_times), seq.preemptions)

    def stop(self) -> None:
        """Finish every live request (reference: ServingEngine.Stop, serving.go:693-709)."""
        self._stopped = True
        for seq in list(self.scheduler.running.values()):
            self.scheduler.finish(seq, "abort")
        while self.scheduler.waiting:
            seq = self.scheduler.waiting.popleft()
            seq.finish_reason = "abort"
            seq.state = SeqState.FINISHED
