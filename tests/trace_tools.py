"""Helpers of the replay tests: make a model folder, build traces that cut the same
requests in different ways, drive bin/trace_run, and compare what it wrote with
the plain implementation."""
import json
import os
import random
import subprocess
import sys

import numpy as np
import torch

import plain_llama

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def round64(n):
    return -(-n // 64) * 64


def random_requests(vocab, lengths, seed):
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(vocab) for _ in range(n)] for i, n in enumerate(lengths)}


class Trace:
    """Steps plus, for every wanted row, which (request, position) it is."""

    def __init__(self):
        self.steps = []
        self.expect = {}          # step -> [(request name, position)]
        self.live = {}            # trace id -> tokens held
        self.totals = {}          # trace id -> tokens it held when it ended (or holds)
        self.peak = 0

    def add(self, entries, end=()):
        """entries: [(trace id, request name, start, tokens, want)]"""
        n = len(self.steps)
        rec = {"step": n, "entries": [], "end": list(end)}
        exp = []
        for tid, name, start, tokens, want in entries:
            rec["entries"].append({"id": tid, "tokens": list(tokens), "want": list(want)})
            exp.extend((name, start + w) for w in want)
            self.live[tid] = self.live.get(tid, 0) + len(tokens)
            self.totals[tid] = self.live[tid]
        self.peak = max(self.peak, sum(round64(v) for v in self.live.values()))
        for tid in end:
            self.live.pop(tid, None)
        self.steps.append(rec)
        if exp:
            self.expect[n] = exp
        return n


def whole(trace, requests, tag="w"):
    for name, toks in requests.items():
        trace.add([(f"{tag}-{name}", name, 0, toks, range(len(toks)))], end=[f"{tag}-{name}"])


def tail_decode(trace, requests, tail=32, tag="d"):
    for name, toks in requests.items():
        tid = f"{tag}-{name}"
        cut = max(1, len(toks) - tail)
        trace.add([(tid, name, 0, toks[:cut], [cut - 1])])
        for p in range(cut, len(toks)):
            trace.add([(tid, name, p, toks[p:p + 1], [0])], end=[tid] if p == len(toks) - 1 else [])
        if cut == len(toks):
            trace.add([], end=[tid])


def portions(trace, requests, sizes=(16, 7, 2, 5, 3, 2, 11, 2, 4, 9, 2, 33, 2), tag="p"):
    for name, toks in requests.items():
        tid, p, i = f"{tag}-{name}", 0, 0
        while p < len(toks):
            n = min(sizes[i % len(sizes)], len(toks) - p)
            if len(toks) - p - n == 1:      # never leave a lone last token: portions go down to two
                n += 1
            i += 1
            last = p + n == len(toks)
            trace.add([(tid, name, p, toks[p:p + n], range(n))], end=[tid] if last else [])
            p += n


def mixed(trace, requests, max_live=4, seed=0, tag="m"):
    """Up to max_live requests at a time: each first takes its prompt in portions of
    changing size, then its last tokens one by one, while others are elsewhere in
    that course.  A request sometimes sits a step out."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live = []                      # [tid, name, toks, pos, decode_from]
    n_started = 0
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.6):
            name, toks = waiting.pop(0)
            dec_from = max(1, len(toks) - rng.choice([3, 8, 17]))
            live.append([f"{tag}{n_started}-{name}", name, toks, 0, dec_from])
            n_started += 1
        entries, ended = [], []
        for item in live:
            tid, name, toks, pos, dec_from = item
            if len(live) > 1 and rng.random() < 0.15:
                continue                              # sits this step out
            if pos < dec_from:
                n = min(rng.choice([2, 3, 5, 8, 16, 21]), dec_from - pos)
                if dec_from - pos - n == 1:
                    n += 1
            else:
                n = 1
            want = list(range(n)) if rng.random() < 0.7 else [n - 1]
            entries.append((tid, name, pos, toks[pos:pos + n], want))
            item[3] = pos + n
            if item[3] == len(toks):
                ended.append(tid)
        if entries:
            trace.add(entries, end=ended)
        live = [it for it in live if it[3] < len(it[2])]


def run_trace(model_dir, dtype, trace, out_dir, block_size=16, extra_args=(), timeout=600, env=None):
    """Drive bin/trace_run: one step a line, waiting for its 'done' before the next.  The
    pool is the trace's peak of live tokens and nothing more; which request held which page
    is logged to <out_dir>/pages.jsonl."""
    os.makedirs(out_dir, exist_ok=True)
    cmd = [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(trace.peak), "--block-size", str(block_size),
           "--debug-pages", os.path.join(out_dir, "pages.jsonl"), *extra_args]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    try:
        for rec in trace.steps:
            proc.stdin.write(json.dumps(rec) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {rec['step']}", f"step {rec['step']}: got {line!r}"
        proc.stdin.close()
        rc = proc.wait(timeout=timeout)
    finally:
        if proc.poll() is None:
            proc.kill()
    assert rc == 0, f"trace_run exited with {rc}"


def pages_were_used_again(trace, page_log_path, block_size):
    """What makes a replay a test of page reuse, asserted instead of assumed: the pool (the
    trace's peak, which is what --max-tokens is given) holds fewer pages than the trace's
    requests take together, and some page id was held by two different requests in the course
    of the trace.  Returns (pool pages, pages of all requests, page ids held by more than one)."""
    pool = -(-trace.peak // 64) * 64 // block_size
    asked = sum(-(-n // block_size) for n in trace.totals.values())
    assert pool < asked, f"the pool of {pool} pages holds all {asked} pages the trace ever asks for"
    owners = {}
    with open(page_log_path) as f:
        for line in f:
            rec = json.loads(line)
            for rid, groups in rec["pages"].items():
                for g, pages in enumerate(groups):
                    for p in pages:
                        if p >= 0:
                            owners.setdefault((g, p), set()).add(rid)
    shared = [k for k, v in owners.items() if len(v) > 1]
    assert shared, "no page was ever held by two different requests"
    return pool, asked, len(shared)


def plain_logits(weights, config, requests):
    return {name: plain_llama.forward(weights, config, toks) for name, toks in requests.items()}


def compare(trace, out_dir, reference, vocab, rel_tol):
    """Every written row against the plain logits of its (request, position).  The
    error of a row is max|diff| / max|reference row|.  Returns the worst."""
    worst, where = 0.0, None
    for step, exp in trace.expect.items():
        path = os.path.join(out_dir, f"{step}.f32")
        assert os.path.exists(path), f"step {step} wrote no file"
        got = np.fromfile(path, dtype="<f4").reshape(-1, vocab)
        assert got.shape[0] == len(exp), f"step {step}: {got.shape[0]} rows, expected {len(exp)}"
        for row, (name, pos) in zip(got, exp):
            ref = reference[name][pos].numpy()
            assert np.isfinite(row).all(), f"step {step} {name}@{pos}: non-finite logits"
            err = float(np.abs(row - ref).max() / max(np.abs(ref).max(), 1e-6))
            if err > worst:
                worst, where = err, (step, name, pos)
    assert worst <= rel_tol, f"worst relative error {worst:.3e} at (step, request, position) {where}"
    return worst


def model_folder(tmp, name, config, seed, std, jitter, dtype="float32"):
    from gollmgo_b200.weights import write_random_model
    d = os.path.join(tmp, name)
    write_random_model(d, config, seed, dtype=dtype, std=std, norm_jitter=jitter)
    return d


def load_weights(model_dir):
    from safetensors.torch import load_file
    return {k: v.to(torch.float32) for k, v in load_file(os.path.join(model_dir, "model.safetensors")).items()}
