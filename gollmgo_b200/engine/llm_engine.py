"""The engine: requests in, tokens out.  One loop ticks the scheduler, builds the
step's batch, runs the step function, samples, and finishes sequences.

Shape of the loop and of the public calls follows the reference's ServingEngine
(internal/engine/serving.go:160-204 loop, 308-461 runStep, 465-490 emit,
670-691 Enqueue, 800-823 cleanup) and its Request{ID, TokenIDs, MaxTokens}
(internal/engine/engine.go:7-11); it runs in the caller's thread instead of a
goroutine: ``step()`` is one turn of the loop, ``generate()`` runs it to the end.

A step that fails (the runner raises, or a kernel reports that it gave up on a
bounded wait) ends the sequences that took part in it with an error result and
gives their pages and state slots back; the queue behind them is served as
before (internal/engine/serving.go:199-202, 646-666 recoverFromStepFailure).
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
from .sequence import PENDING, SeqState, Sequence


@dataclass
class TokenResult:
    """One generated token (the reference's TokenResult: internal/engine/engine.go:14-20)."""
    request_id: str
    token_id: int
    finished: bool
    finish_reason: Optional[str] = None
    error: Optional[str] = None          # set on the last result of a request whose step failed (token_id -1)


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
    error: Optional[str] = None          # finish_reason "error": what failed


@dataclass
class EngineStats:
    steps: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    generated_tokens: int = 0
    preemptions: int = 0
    pages_high_water: int = 0
    failed_steps: int = 0
    failed_requests: int = 0
    batch_sum: int = 0                   # sequences over all steps (mean batch = batch_sum / steps)


class Engine:
    def __init__(self, model: Optional[str] = None, *, config: Optional[dict] = None,
                 weights_seed: Optional[int] = None, engine_config: Optional[EngineConfig] = None,
                 runner=None, sampler=None, **engine_options):
        """``model``: a folder with config.json and *.safetensors.  Or ``config`` (a
        config.json dict) with ``weights_seed`` for random weights made on the device.
        Engine options (EngineConfig fields) may be given as keywords.

        ``runner`` and ``sampler`` replace the step function and the token selection with
        objects of the caller's (the runner: ``spec``, ``cache``, ``max_model_len``, ``device``,
        ``last_tokens``, ``step(entries)``, ``check_kernels()``; the sampler: ``sample_async``,
        ``wait``): the loop, the scheduler and the failure handling can then be driven without
        a device, which is how the tests inject a step that fails."""
        ecfg = engine_config or EngineConfig(**engine_options)
        if runner is not None:
            self.runner = runner
        elif model is not None:
            self.runner = ModelRunner(read_config_json(model), ecfg, weights=model)
        elif config is not None:
            self.runner = ModelRunner(config, ecfg, weights_seed=weights_seed if weights_seed is not None else 0)
        else:
            raise ValueError("give a model folder, or a config with weights_seed")
        self.ecfg = ecfg
        self.spec = self.runner.spec
        self.scheduler = Scheduler(ecfg, self.runner.cache, self.runner.max_model_len)
        if sampler is not None:
            self.sampler = sampler
        else:
            from ..sampling.sampler import Sampler
            self.sampler = Sampler(self.runner.device, max(ecfg.max_batch_size, 1), self.runner.last_tokens)
        self._inflight = None
        self.sequences: Dict[str, Sequence] = {}
        self.stats = EngineStats()
        self._next_id = 0
        self._seed_rng = random.Random()
        self._stopped = False
        if ecfg.cuda_graphs and ecfg.capture_at_start and hasattr(self.runner, "capture_graphs"):
            self.runner.capture_graphs()

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
        if len(token_ids) and not (0 <= min(token_ids) and max(token_ids) < V):
            bad = next(t for t in token_ids if not (0 <= int(t) < V))
            raise ValueError(f"token id {bad} is outside [0, {V})")
        seq_id = self._next_id
        self._next_id += 1
        rid = request_id if request_id is not None else f"req-{seq_id}"
        if rid in self.sequences and not self.sequences[rid].finished:
            raise ValueError(f"request id {rid!r} is in use")
        seq = Sequence(seq_id, rid, [int(t) for t in token_ids], params)
        self.scheduler.add(seq)
        self.sequences[rid] = seq
        return rid

    # ------------------------------------------------------------------ one turn of the loop
    def step(self) -> List[TokenResult]:
        """One turn: plan and launch the next step, then hand out the tokens of the step
        launched one turn earlier.

        The device runs one step ahead of the host.  A sequence that sampled in the step
        still in flight gets a placeholder for its unknown token; the step launched now
        reads that token on the device (from the sampler's buffer), so the host work of
        this turn overlaps the device's work on the step before.  What the host cannot
        know one step early is an end-of-sequence token: such a sequence takes part in
        one step too many, whose token is dropped.  Finishing by length is known early.
        """
        plan: SchedulerOutput = self.scheduler.schedule()
        self.stats.preemptions += len(plan.preempted)
        launched = None
        results: List[TokenResult] = []
        if plan.scheduled:
            entries, samplers = [], []
            for s in plan.scheduled:
                seq = s.seq
                toks = seq.token_slice(seq.num_computed, seq.num_computed + s.num_tokens)
                src = -1
                if toks[-1] == PENDING:
                    if s.num_tokens != 1:
                        raise RuntimeError("a token still on the device can only be fed alone")
                    toks, src = [0], seq.pending_row
                if PENDING in toks:
                    raise RuntimeError("an unknown token in the middle of a portion")
                entries.append(StepEntry(seq.id, toks, [s.num_tokens - 1] if s.samples else [], src, checked=True))
                if s.samples:
                    samplers.append(seq)
            try:
                logits = self.runner.step(entries)
                handle = self.sampler.sample_async(logits, [q.params for q in samplers],
                                                   [len(q.output) for q in samplers])
            except Exception as exc:          # noqa: BLE001  (whatever the step function raises)
                # the step did not run: first hand out what the step before produced (those
                # tokens are good), then end the sequences of this one
                inflight, self._inflight = self._inflight, None
                try:
                    results = self._resolve(inflight)
                except Exception as exc2:     # noqa: BLE001
                    results = self._fail(inflight[2], exc2)
                results += self._fail([s.seq for s in plan.scheduled], exc)
                return results
            for s in plan.scheduled:
                self.scheduler.advance(s)
            for row, seq in enumerate(samplers):
                seq.output.append(PENDING)
                seq.pending_row = row
                self.scheduler.token_sampled(seq)
                if len(seq.output) >= seq.params.max_tokens:
                    self.scheduler.finish(seq, "length")          # known without the token's value
            launched = (handle, samplers, [s.seq for s in plan.scheduled])
            st = self.stats
            st.steps += 1
            st.batch_sum += len(plan.scheduled)
            st.prefill_tokens += plan.prefill_tokens
            st.decode_tokens += plan.decode_tokens
            st.pages_high_water = max((g.pool.high_water for g in self.runner.cache.groups), default=0)
        elif self._inflight is None and self.scheduler.has_work() and not plan.preempted:
            raise RuntimeError("scheduler made no progress: the page pool is too small for the "
                               "request at the head of the queue")
        inflight, self._inflight = self._inflight, launched
        try:
            results = self._resolve(inflight)
        except Exception as exc:              # noqa: BLE001
            # the step before turned out to have failed (a kernel gave up on a bounded wait, the
            # copy of its tokens did not arrive).  The step launched in this turn read its cache
            # and its tokens, so it is void as well.
            results = self._fail(inflight[2] + (launched[2] if launched else []), exc)
            self._drain(launched)
            self._inflight = None
        return results

    def _drain(self, launched) -> None:
        """Wait for a launched step whose results will not be used."""
        if launched is None:
            return
        try:
            self.sampler.wait(launched[0])
            self.runner.check_kernels()
        except Exception:                     # noqa: BLE001  (it is void either way)
            pass

    def _fail(self, seqs, exc) -> List[TokenResult]:
        """End the sequences of a failed step: placeholders of tokens that will never be read
        are dropped, pages and state slots go back, each gets one last result that carries the
        error.  A sequence that had ended already with every token known is left alone."""
        msg = f"{type(exc).__name__}: {exc}"
        self.stats.failed_steps += 1
        results = []
        seen = set()
        for seq in seqs:
            if seq.id in seen or (seq.finished and seq.resolved == len(seq.output)):
                continue
            seen.add(seq.id)
            del seq.output[seq.resolved:]
            seq.dropped = True
            seq.error = msg
            seq.num_computed = 0
            self.scheduler.finish(seq, "error")
            self.stats.failed_requests += 1
            results.append(TokenResult(seq.request_id, -1, True, "error", msg))
        return results

    def _resolve(self, inflight) -> List[TokenResult]:
        """Read the tokens of a launched step and settle its sequences."""
        if inflight is None:
            return []
        handle, samplers = inflight[0], inflight[1]
        tokens = self.sampler.wait(handle)
        self.runner.check_kernels(wait=False)      # this step's status has arrived with its tokens; a step launched since is not waited for
        now = time.perf_counter()
        eos = set(self.spec.eos_token_ids)
        results = []
        for seq, tok in zip(samplers, tokens):
            if seq.dropped:                    # ended by an earlier token; this one was one step too many
                continue
            tok = int(tok)
            idx = seq.resolved
            seq.output[idx] = tok
            seq.resolved += 1
            seq.token_times.append(now)
            if seq.first_token_at is None:
                seq.first_token_at = now
            seq.last_token_at = now
            reason = None
            if not seq.params.ignore_eos and tok in eos:
                reason = "stop"
                del seq.output[idx + 1:]       # a placeholder of the step launched since
                seq.dropped = True
                # wherever it is by now: running, ended by length at launch, or back in the
                # queue because it was preempted while this token was on its way
                self.scheduler.finish(seq, "stop")
            elif seq.resolved >= seq.params.max_tokens:
                reason = "length"
            results.append(TokenResult(seq.request_id, tok, reason is not None, reason))
            self.stats.generated_tokens += 1
        return results

    def has_unfinished(self) -> bool:
        return self.scheduler.has_work() or self._inflight is not None

    add_request = enqueue

    def replay(self, lines, out_dir: str) -> int:
        """Trace replay (engine/trace.py) on this engine's runner: ``lines`` is an iterable of
        JSON steps; logits at the wanted places are written to ``out_dir``.  Returns the
        number of steps.  Use it on an engine with no requests of its own in flight."""
        from .trace import replay
        if self.has_unfinished():
            raise RuntimeError("replay needs an idle engine")
        import io
        return replay(self.runner, lines, out_dir, log=io.StringIO())

    # ------------------------------------------------------------------ whole requests
    def generate(self, prompts: Seq[Seq[int]], params=None, concurrency: int = 0,
                 **param_options) -> List[RequestOutput]:
        """Generate for every prompt (token ids); returns outputs in the order given.
        ``params``: one SamplingParams for all, or one per prompt.  ``concurrency`` > 0: a closed
        loop, as the reference's serving benchmark drives its server (bench/PARITY_SUMMARY.md:
        concurrency 4): at most that many requests are in the engine at a time, and the next
        prompt is handed in when one of them has finished; 0: all at once."""
        if params is None:
            params = SamplingParams(**param_options)
        plist = list(params) if isinstance(params, (list, tuple)) else [params] * len(prompts)
        if len(plist) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        if concurrency < 0:
            raise ValueError("concurrency must be 0 (all at once) or a positive number of requests")
        rids = []
        pending = list(zip(prompts, plist))
        i, live = 0, 0
        while i < len(pending) or self.has_unfinished():
            while i < len(pending) and (concurrency <= 0 or live < concurrency) and (
                    self.ecfg.max_queue_depth <= 0 or len(self.scheduler.waiting) < self.ecfg.max_queue_depth):
                rids.append(self.enqueue(pending[i][0], pending[i][1]))
                i += 1
                live += 1
            live -= sum(1 for r in self.step() if r.finished)
        return [self.output_of(r) for r in rids]

    def output_of(self, request_id: str) -> RequestOutput:
        seq = self.sequences[request_id]
        return RequestOutput(seq.request_id, list(seq.prompt), list(seq.output), seq.finish_reason,
                             (seq.first_token_at - seq.created_at) if seq.first_token_at else None,
                             (seq.last_token_at - seq.created_at) if seq.last_token_at else None,
                             list(seq.token_times), seq.preemptions, seq.error)

    def stop(self) -> None:
        """Finish every live request (reference: ServingEngine.Stop, serving.go:693-709)."""
        self._stopped = True
        self._resolve(self._inflight)
        self._inflight = None
        for seq in list(self.scheduler.running.values()):
            self.scheduler.finish(seq, "abort")
        while self.scheduler.waiting:
            seq = self.scheduler.waiting.popleft()
            seq.finish_reason = "abort"
            seq.state = SeqState.FINISHED
