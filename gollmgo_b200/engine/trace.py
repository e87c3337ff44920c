"""Trace replay: feed given token ids through the model step by step and write the
logits at the wanted places.  Nothing is sampled.  It drives the same runner,
step function, cache manager and kernels that generation uses; it has no forward
pass, cache or loader of its own.  (The reference has no such tool; the nearest is
the manual RunStep of internal/engine/inference.go:66-139.)

A step is one JSON object on a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step that wants something, ``<out>/<step>.f32`` holds the logits
[wanted places, vocab] as little-endian float32, in the order of the entries and
of each entry's ``want``.  After every step ``done <step>`` is printed.
"""
from __future__ import annotations

import json
import os
import sys
from typing import IO, List

import torch

from ..config import EngineConfig, read_config_json
from .batch import StepEntry
from .runner import ModelRunner

PAGE_ROUND = 64          # a request's token count is rounded up to this in --max-tokens


def make_trace_runner(model_dir: str, dtype: str, max_tokens: int, block_size: int = 16,
                      max_live: int = 4, token_budget: int = 8192, cuda_graphs: bool = True) -> ModelRunner:
    if PAGE_ROUND % block_size:
        raise ValueError(f"page size {block_size} does not divide {PAGE_ROUND}")
    max_tokens = max(PAGE_ROUND, -(-max_tokens // PAGE_ROUND) * PAGE_ROUND)
    ecfg = EngineConfig(dtype=dtype, block_size=block_size, num_blocks=max_tokens // block_size,
                        max_batch_size=max(2 * max_live, 8),
                        max_token_budget=min(token_budget, max_tokens),
                        max_model_len=max_tokens, cuda_graphs=cuda_graphs)
    return ModelRunner(read_config_json(model_dir), ecfg, weights=model_dir)


def run_step(runner: ModelRunner, entries: List[StepEntry]) -> torch.Tensor:
    """One trace step of any size: cut into sub-steps that fit the runner's token
    budget (a cut changes nothing but rounding), logits gathered in order."""
    budget = runner.ctx.max_tokens
    if sum(len(e.tokens) for e in entries) <= budget:
        return runner.step(entries)
    # place of each wanted row in the final order
    order, n = {}, 0
    for ei, e in enumerate(entries):
        for w in e.want:
            order[(ei, w)] = n
            n += 1
    out = torch.empty(n, runner.spec.vocab_size, dtype=torch.float32, device=runner.device)
    progress = [0] * len(entries)
    while any(p < len(e.tokens) for p, e in zip(progress, entries)):
        room, sub, keys = budget, [], []
        for ei, e in enumerate(entries):
            if room == 0 or progress[ei] >= len(e.tokens):
                continue
            lo = progress[ei]
            hi = min(len(e.tokens), lo + room)
            want = [w - lo for w in e.want if lo <= w < hi]
            keys.extend((ei, w) for w in e.want if lo <= w < hi)
            sub.append(StepEntry(e.request_id, list(e.tokens[lo:hi]), want))
            progress[ei] = hi
            room -= hi - lo
        logits = runner.step(sub)
        for i, k in enumerate(keys):
            out[order[k]] = logits[i]
    return out


def replay(runner: ModelRunner, lines: IO[str], out_dir: str, log: IO[str] = sys.stdout,
           page_log: IO[str] = None) -> int:
    """Run the steps read from ``lines``.  ``page_log``: after every step one JSON line
    {"step": n, "pages": {request id: [page ids of group 0, of group 1, ...]}} for the requests
    of that step, so that a test can see which request held which page when (-1 = a page that a
    sliding group has given back)."""
    os.makedirs(out_dir, exist_ok=True)
    steps = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = [StepEntry(e["id"], [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])])
                   for e in rec.get("entries", [])]
        if entries:
            logits = run_step(runner, entries)
            if logits.shape[0]:
                data = logits.to("cpu", torch.float32).contiguous().numpy()
                data.astype("<f4", copy=False).tofile(os.path.join(out_dir, f"{step}.f32"))
            else:
                torch.cuda.synchronize(runner.device)
            runner.check_kernels()
            if page_log is not None:
                held = {str(e.request_id): [list(map(int, runner.cache.block_table(e.request_id, g)))
                                            for g in range(len(runner.cache.groups))] for e in entries}
                page_log.write(json.dumps({"step": step, "pages": held}) + "\n")
                page_log.flush()
        for rid in rec.get("end", []):
            if runner.has(rid):
                runner.release(rid)
        print(f"done {step}", file=log, flush=True)
        steps += 1
    return steps
