"""The step function: run a batch of (request, its next tokens) through the model,
from the cache, and return the logits at the wanted places.

``ModelRunner`` owns the model, the cache manager and the batch builder.  A step
runs only the tokens it is given, as one batch; what earlier steps left in the
cache is what those tokens attend to.  Steps that hold one token per sequence
can be captured in a CUDA graph per batch bucket and replayed: every size a
kernel reads that changes between steps (context lengths, block tables, slots)
lives in device memory.

Reference: Runner.Step (internal/backend/runner.go:83-92) and
CUDARunnerWithModel.Step (internal/backend/cuda/model_bridge.go:207-239); its
decode graph is keyed by (batch, longest context) and re-captured as contexts
grow (kernels/gollmgo_model.cu:1004-1054).
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence

import torch

from .. import architectures  # noqa: F401  (registers the architectures)
from ..cache import CacheManager, OutOfPages, PagedKVNeed
from ..config import EngineConfig, read_config_json
from ..csrc import ops
from ..parts import BuildContext, StepFacts, build_model, set_matmul_precision
from ..weights import checkpoint_source, random_source
from .batch import BatchBuilder, StepBatch, StepEntry

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}
GRAPH_BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)


class ModelRunner:
    def __init__(self, config_dict: dict, engine_config: EngineConfig, weights=None,
                 weights_seed: Optional[int] = None):
        """``weights``: a model folder; or ``weights_seed``: random weights on the device."""
        engine_config.validate()
        if not torch.cuda.is_available():
            raise RuntimeError("gollmgo_b200 runs on a CUDA device (sm_100a); none is visible")
        self.ecfg = engine_config
        self.device = torch.device("cuda", engine_config.device)
        torch.cuda.set_device(self.device)
        cap = ops.device_capability()          # loads (and if needed builds) the CUDA library
        if cap < 100:
            raise RuntimeError(f"the kernels are built for sm_100a; this device is sm_{cap}")
        set_matmul_precision()
        self.dtype = _DTYPES[engine_config.dtype]
        max_tokens = engine_config.max_token_budget
        ctx = BuildContext(self.dtype, self.device, max_tokens, engine_config.max_batch_size,
                           engine_config.block_size)
        self.ctx = ctx
        self.config, self.spec, self.model = build_model(config_dict, ctx)
        manifest = self.model.manifest()
        if weights is not None:
            get = checkpoint_source(weights, manifest, self.dtype, self.device)
        elif weights_seed is not None:
            get = random_source(manifest, weights_seed, self.device, self.dtype)
        else:
            raise ValueError("give a model folder or a seed for random weights")
        self.model.load(get)
        self.max_model_len = engine_config.max_model_len or self.spec.max_positions
        needs = self.model.cache_needs()
        self.num_pages = engine_config.num_blocks or self._pages_from_memory(needs)
        self.cache = CacheManager(needs, engine_config.block_size, self.num_pages,
                                  max_requests=max(engine_config.max_batch_size, 4) * 2,
                                  dtype=self.dtype, device=self.device)
        self.caches = [self._cache_view(i, n) for i, n in enumerate(needs)]
        self.builder = BatchBuilder(self.cache, self.device, query_tiles=self.model.query_tiles())
        # tokens sampled on the device in the last step, by row: the next step may take its
        # inputs from here before the host has read them
        self.last_tokens = torch.zeros(max(engine_config.max_batch_size, 1), dtype=torch.int32,
                                       device=self.device)
        # the status word of the tcgen05 kernels, copied to the host behind every step that ran one
        # (two steps can be in flight), so that reading it never waits for a step launched since
        self._status_host = [torch.zeros(1, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._status_event = [torch.cuda.Event(), torch.cuda.Event()]
        self._status_pending = [False, False]
        self._status_turn = 0
        self._graphs: Dict[int, "_CapturedStep"] = {}
        self.steps = 0
        self.launch_count = 0

    # ------------------------------------------------------------------ set-up
    def _pages_from_memory(self, needs) -> int:
        """Pages per group from the memory left after weights and workspace
        (reference sizing: cmd/gollmgo/gpu.go:151-177)."""
        per_page = CacheManager.bytes_per_page(needs, self.ecfg.block_size,
                                               torch.empty((), dtype=self.dtype).element_size())
        # every layer of a group shares the page id, so one page id costs per_page per layer;
        # bytes_per_page already sums over cache entries
        free, _ = torch.cuda.mem_get_info(self.device)
        reserve = self.ctx.workspace.nbytes() + (512 << 20)
        avail = int((free - reserve) * self.ecfg.max_memory_fraction)
        if per_page <= 0:
            return 64
        return max(64, avail // per_page)

    def _cache_view(self, cache_id: int, need):
        if isinstance(need, PagedKVNeed):
            return self.cache.layer_cache(cache_id)
        if need is None:
            return None
        return self.cache.state_buffers[cache_id]

    # ------------------------------------------------------------------ requests
    def admit(self, request_id) -> None:
        self.cache.admit(request_id)

    def release(self, request_id) -> None:
        self.cache.free(request_id)

    def has(self, request_id) -> bool:
        return request_id in self.cache.requests

    # ------------------------------------------------------------------ the step
    def _validate(self, entries: Sequence[StepEntry]) -> None:
        V = self.spec.vocab_size
        total = 0
        for e in entries:
            total += len(e.tokens)
            if not e.checked:
                for t in e.tokens:
                    if not (0 <= int(t) < V):
                        raise ValueError(f"request {e.request_id!r}: token id {t} is outside [0, {V})")
            if e.request_id in self.cache.requests and \
                    self.cache.num_tokens(e.request_id) + len(e.tokens) > self.max_model_len:
                raise ValueError(f"request {e.request_id!r} would exceed max_model_len "
                                 f"{self.max_model_len}")
        if total > self.ctx.max_tokens:
            raise ValueError(f"step of {total} tokens exceeds max_token_budget {self.ctx.max_tokens}")
        if len(entries) > self.ctx.max_seqs:
            raise ValueError(f"step of {len(entries)} sequences exceeds max_batch_size {self.ctx.max_seqs}")

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run one batch.  Requests not seen before are admitted.  Returns float32
        logits [wanted places, vocab] on the device, in the order of the entries
        and of each entry's ``want``."""
        self._validate(entries)
        admitted, starts = [], {}
        try:
            for e in entries:
                if e.request_id not in self.cache.requests:
                    self.cache.admit(e.request_id)
                    admitted.append(e.request_id)
                starts[e.request_id] = self.cache.num_tokens(e.request_id)
            logits = self._run(entries)
            if ops.tc_launched:
                self._snapshot_status()
            return logits
        except Exception:
            # a step that fails leaves nothing behind: no token of it counts as cached (what a
            # kernel may have written lies beyond every request's count and is overwritten by
            # the tokens that come there next), and requests it admitted are gone again
            for rid, n in starts.items():
                if rid in self.cache.requests and self.cache.num_tokens(rid) > n:
                    self.cache.rollback(rid, n)
            for rid in admitted:
                if rid in self.cache.requests:
                    self.cache.free(rid)
            raise

    def _run(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        decode_only = all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)
        # The model's parts may tag the step from what is known before its batch is built (the
        # attention: some live request holds a long context).  Steps with different tags are steps
        # of different kinds: a part may choose differently for them, so each kind has captured
        # graphs of its own.  The runner only carries the tags; it does not know what they mean.
        n_tokens, longest = sum(len(e.tokens) for e in entries), int(self.cache.ntok.max())
        if decode_only and self.ecfg.cuda_graphs:
            bucket = next((b for b in GRAPH_BUCKETS if b >= len(entries)), None)
            if bucket is not None and bucket <= self.ctx.max_seqs:
                # a captured step runs the bucket's number of sequences (the rest are padding)
                facts = StepFacts(bucket, bucket, True, longest)
                return self._graph_step(entries, bucket, facts, self.model.step_tags(facts))
        facts = StepFacts(len(entries), n_tokens, decode_only, longest)
        batch = self.builder.build(entries)
        batch.facts, batch.tags = facts, self.model.step_tags(facts)
        batch.prev_tokens = self.last_tokens if batch.token_src is not None else None
        logits = self.model.forward(batch, self.caches)
        self.steps += 1
        return logits

    def _snapshot_status(self) -> None:
        ops.tc_launched = False
        slot = self._status_turn
        self._status_turn ^= 1
        if self._status_pending[slot]:                  # a snapshot nobody asked about: it still counts
            self._read_status(slot)
        self._status_host[slot].copy_(ops.tc_status(self.device), non_blocking=True)
        self._status_event[slot].record()
        self._status_pending[slot] = True

    def _read_status(self, slot: int) -> None:
        self._status_event[slot].synchronize()
        self._status_pending[slot] = False
        code = int(self._status_host[slot][0])
        if code:
            ops.tc_status(self.device).zero_()
            raise ops.KernelError(f"a tcgen05 kernel gave up waiting on a barrier (code {code}); the step's output is not valid")

    def check_kernels(self, wait: bool = True) -> None:
        """Raise if a kernel of a step reported that it gave up on a bounded wait.  The status
        word travels to the host behind each step (a copy in stream order), so asking about a
        step whose results the host has already read costs nothing.  ``wait=False``: only ask
        about steps whose copy has arrived (a step launched since is left for the next call)."""
        for slot in (self._status_turn, self._status_turn ^ 1):          # the older one first
            if self._status_pending[slot] and (wait or self._status_event[slot].query()):
                self._read_status(slot)

    # ------------------------------------------------------------------ captured decode steps
    def _graph_stride(self) -> int:
        return -(-self.max_model_len // self.cache.page_size)

    def _graph_step(self, entries, bucket: int, facts: StepFacts, tags: tuple = ()) -> torch.Tensor:
        key = (bucket, tags) if tags else bucket
        cs = self._graphs.get(key)
        stride = self._graph_stride()
        if cs is None:
            lay = self.builder.decode_layout(bucket, stride)
            cs = _CapturedStep(torch.zeros(lay.size, dtype=torch.int32, device=self.device))
            self._graphs[key] = cs
        batch = self.builder.build(entries, fixed_seqs=bucket, fixed_stride=stride, static_dev=cs.meta)
        batch.facts, batch.tags = facts, tags
        batch.prev_tokens = self.last_tokens
        if cs.graph is None:
            torch.cuda.synchronize(self.device)
            # warm-up on a side stream, then capture
            s = torch.cuda.Stream(self.device)
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self.model.forward(batch, self.caches)
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            before = ops.launches
            with torch.cuda.graph(g):
                cs.logits = self.model.forward(batch, self.caches)
            cs.launches = ops.launches - before
            cs.graph = g
        cs.graph.replay()
        ops.launches += cs.launches
        self.steps += 1
        return cs.logits[:len(entries)]

    def capture_graphs(self, up_to: Optional[int] = None) -> int:
        """Capture now the decode step of every batch bucket up to ``up_to`` sequences (default:
        the largest batch), in every kind that the model's parts tell apart as contexts grow to
        the longest sequence allowed (the tags of ``step_tags`` for contexts of 1, 2, 4, ...
        tokens), so that no request meets the tens of milliseconds of a capture in the middle of
        its generation when the batch or its context grows into a new kind for the first time.
        Uses a request of its own of a few tokens and gives its page back.  Returns the number
        of steps captured."""
        if not self.ecfg.cuda_graphs or self.device.type != "cuda":
            return 0
        rid = "__capture__"
        limit = min(up_to or self.ctx.max_seqs, self.ctx.max_seqs)
        contexts, c = [], 1
        while c < 2 * self.max_model_len:
            contexts.append(min(c, self.max_model_len))
            c *= 2
        todo = []
        for bkt in (b for b in GRAPH_BUCKETS if b <= limit):
            for c in contexts:
                facts = StepFacts(bkt, bkt, True, c)
                tags = self.model.step_tags(facts)
                key = (bkt, tags) if tags else bkt
                if (key not in self._graphs or self._graphs[key].graph is None) and all(k != key for k, _, _ in todo):
                    todo.append((key, facts, tags))
        if not todo or len(todo) + 1 > self.max_model_len:
            return 0
        marks = [g.pool.high_water for g in self.cache.groups]
        self.cache.admit(rid)
        done = 0
        try:
            for key, facts, tags in todo:
                if self.cache.num_tokens(rid) + 1 >= self.max_model_len:       # the request is full: start it again
                    self.cache.free(rid)
                    self.cache.admit(rid)
                self._graph_step([StepEntry(rid, [0], [0])], facts.num_seqs, facts, tags)
                done += 1
            torch.cuda.synchronize(self.device)
        except OutOfPages:
            pass                                   # a pool too small even for this: capture at first use instead
        finally:
            if rid in self.cache.requests:
                self.cache.free(rid)
            for g, m in zip(self.cache.groups, marks):
                g.pool.high_water = m
        return done

    # ------------------------------------------------------------------ facts
    def memory_report(self) -> dict:
        return {"weights_bytes": self.model.weight_bytes(),
                "workspace_bytes": self.ctx.workspace.nbytes(),
                "cache_pages": self.num_pages, "page_size": self.cache.page_size}


class _CapturedStep:
    def __init__(self, meta: torch.Tensor):
        self.meta = meta
        self.graph = None
        self.logits = None
        self.launches = 0


def load_runner(model_dir: str, engine_config: EngineConfig) -> ModelRunner:
    """Runner for the model in ``model_dir`` (config.json + *.safetensors)."""
    return ModelRunner(read_config_json(model_dir), engine_config, weights=model_dir)
