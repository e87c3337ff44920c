"""The layer sizes of the headline configuration (hidden 4096, 32/8 heads of 128, feed-forward
14336, vocabulary 128256, llama3 rope scaling over 8192 positions; two layers, random weights)
against the PLAIN implementation, which runs in float64 on the device for these sizes.

The tiny configurations cannot reach what only these sizes take: several waves of tiles in the
tcgen05 kernels, the weight-streaming products over long rows, 16 KB rows in the norm, the
stacked q/k/v weights at four heads per group, the rope table at its real scaling factors.
The same requests are replayed whole, with the last 32 tokens one by one, in portions down to
two tokens, mixed with other requests on a pool so small that pages are used again, and as
decode-only steps of 64, 40 and 24 sequences with ragged contexts (the steps that take the
swapped-operand tcgen05 products, the library between 33 and 64 tokens, the graph buckets
above 16 and the decode attention for large batches).  Float32 and bfloat16.

The steps go through engine/trace.py::replay in this process (the program bin/trace_run is the
same function behind a command line; the tiny configurations are replayed through it)."""
import io
import json
import os
import random

import pytest
import torch

import plain_llama
import trace_tools as tt

pytestmark = pytest.mark.gpu

SHAPE = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                     "gollmgo_b200", "bench_shapes", "llama_3_1_8b.json")
TOL = {"float32": 1e-4, "bfloat16": 4e-2}
LONG = {"L0": 1500, "L1": 640}                      # whole, tail, portions
SHORT = {"S0": 300, "S1": 77, "S2": 130, "S3": 210, "S4": 64}      # mixed
N_DECODE, DECODE_STEPS = 64, 6


def sparse(n, every=97):
    return sorted(set(range(0, n, every)) | {n - 1})


def build_trace(requests):
    """One trace for everything; returns it with the step index where each part starts."""
    t = tt.Trace()
    parts = {}
    longs = {k: requests[k] for k in LONG}
    parts["whole"] = len(t.steps)
    for name, toks in longs.items():
        t.add([(f"w-{name}", name, 0, toks, sparse(len(toks)))], end=[f"w-{name}"])
    parts["tail"] = len(t.steps)
    for name, toks in longs.items():
        cut = len(toks) - 32
        tid = f"d-{name}"
        t.add([(tid, name, 0, toks[:cut], [cut - 1])])
        for p in range(cut, len(toks)):
            t.add([(tid, name, p, toks[p:p + 1], [0])], end=[tid] if p == len(toks) - 1 else [])
    parts["portions"] = len(t.steps)
    sizes = (1100, 128, 100, 2, 70, 33, 2, 17, 2, 5, 41)
    for name, toks in longs.items():
        tid, p, i = f"p-{name}", 0, 0
        keep = set(sparse(len(toks)))
        while p < len(toks):
            n = min(sizes[i % len(sizes)], len(toks) - p)
            if len(toks) - p - n == 1:
                n += 1
            i += 1
            want = sorted({w - p for w in keep if p <= w < p + n} | {0, n - 1})
            t.add([(tid, name, p, toks[p:p + n], want)], end=[tid] if p + n == len(toks) else [])
            p += n
    parts["mixed"] = len(t.steps)
    tt.mixed(t, {k: requests[k] for k in SHORT}, max_live=4, seed=3)
    parts["decode"] = len(t.steps)
    # decode-only steps of 64, then 40, then 24 sequences: prompts first (eight at a time,
    # prompt portions of different requests in one step), then single tokens
    names = [f"D{i}" for i in range(N_DECODE)]
    for g in range(0, N_DECODE, 8):
        t.add([(f"b-{n}", n, 0, requests[n][:-DECODE_STEPS], [len(requests[n]) - DECODE_STEPS - 1])
               for n in names[g:g + 8]])
    live = list(names)
    for s in range(DECODE_STEPS):
        ended = []
        if s == 1:
            ended = live[40:]
        elif s == 3:
            ended = live[24:]
        elif s == DECODE_STEPS - 1:
            ended = list(live)
        entries = []
        for n in live:
            p = len(requests[n]) - DECODE_STEPS + s
            entries.append((f"b-{n}", n, p, requests[n][p:p + 1], [0]))
        t.add(entries, end=[f"b-{n}" for n in ended])
        live = [n for n in live if n not in ended]
    return t, parts


@pytest.fixture(scope="module")
def big(tmp_path_factory, cuda_device):
    from gollmgo_b200.weights import write_random_model
    with open(SHAPE) as f:
        cfg = json.load(f)
    cfg["num_hidden_layers"] = 2
    tmp = str(tmp_path_factory.mktemp("big"))
    model_dir = write_random_model(os.path.join(tmp, "m"), cfg, seed=5, dtype="bfloat16", std=0.02,
                                   norm_jitter=0.1, device=cuda_device)
    weights = tt.load_weights(model_dir)                   # float32 copies of the bfloat16 checkpoint, on the host
    rng = random.Random(9)
    V = cfg["vocab_size"]
    lengths = dict(LONG)
    lengths.update(SHORT)
    lengths.update({f"D{i}": rng.choice([3, 9, 17, 40, 63, 64, 65, 100, 129, 200]) + DECODE_STEPS
                    for i in range(N_DECODE)})
    requests = {name: [rng.randrange(V) for _ in range(n)] for name, n in lengths.items()}
    trace, parts = build_trace(requests)
    # the plain logits at exactly the places some step wants
    places = {}
    for exp in trace.expect.values():
        for name, pos in exp:
            places.setdefault(name, set()).add(pos)
    reference = {}
    for name, pos in places.items():
        rows = sorted(pos)
        out = plain_llama.forward(weights, cfg, requests[name], device=cuda_device, rows=rows)
        reference[name] = dict(zip(rows, out.to(torch.float32).cpu()))
    torch.cuda.empty_cache()
    return cfg, model_dir, requests, trace, parts, reference


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_cut_and_decode_batches_to_64_match_plain_at_full_width(big, tmp_path, dtype):
    from gollmgo_b200.engine.trace import make_trace_runner, replay
    cfg, model_dir, requests, trace, parts, reference = big
    # the pool holds the peak of live tokens (each request rounded up to 64), nothing more
    runner = make_trace_runner(model_dir, dtype, trace.peak, block_size=16, max_live=N_DECODE // 2,
                               token_budget=2048)
    assert runner.ctx.max_seqs >= N_DECODE
    out = str(tmp_path / "out")
    lines = [json.dumps(rec) for rec in trace.steps]
    with open(out + ".pages", "w") as page_log:
        assert replay(runner, lines, out, log=io.StringIO(), page_log=page_log) == len(trace.steps)
    pool, asked, shared = tt.pages_were_used_again(trace, out + ".pages", 16)
    runner.cache.audit()
    assert not runner.cache.requests and runner.cache.free_pages() == runner.num_pages
    if dtype == "bfloat16":
        # the decode-only steps were captured steps of the buckets they fall into
        assert {64, 48, 24} <= {k[0] if isinstance(k, tuple) else k for k, g in runner._graphs.items() if g.graph is not None}
    V = cfg["vocab_size"]
    worst = {}
    order = sorted(parts, key=parts.get)
    for i, part in enumerate(order):
        lo = parts[part]
        hi = parts[order[i + 1]] if i + 1 < len(order) else len(trace.steps)
        sub = tt.Trace()
        sub.expect = {s: e for s, e in trace.expect.items() if lo <= s < hi}
        assert sub.expect
        worst[part] = tt.compare(sub, out, reference, V, TOL[dtype])
    # greedy choice: where the plain logits have a clear winner, the engine picks it too
    import numpy as np
    checked = 0
    for step, exp in trace.expect.items():
        got = np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4").reshape(-1, V)
        for row, (name, pos) in zip(got, exp):
            ref = reference[name][pos]
            top = torch.topk(ref, 2).values
            if float(top[0] - top[1]) > 2.5 * TOL[dtype] * float(ref.abs().max()):
                assert int(row.argmax()) == int(ref.argmax()), f"step {step} {name}@{pos}"
                checked += 1
    assert checked > 50
    print(f"{dtype}: {len(trace.steps)} steps, pool {pool} pages for {asked} asked, {shared} used again, worst relative error by part "
          + ", ".join(f"{k} {v:.1e}" for k, v in worst.items()) + f"; {checked} greedy choices agree")
