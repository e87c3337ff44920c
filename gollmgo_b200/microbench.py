"""Kernel micro-benchmarks: one kernel at the sizes of a model, timed with CUDA events
on inputs larger than L2 (a ring of weight copies, or a cache of many sequences).

    python -m gollmgo_b200.microbench gemm_small_m [--tokens 8] [--reps 40]
    python -m gollmgo_b200.microbench gemm_tc      [--tokens 2048]
    python -m gollmgo_b200.microbench attn_decode  [--batch 64] [--context 2048]
    python -m gollmgo_b200.microbench attn_prefill [--tokens 2048]
    python -m gollmgo_b200.microbench step_timeline [--batch 8] [--context 2048] [--prompt-tokens 0]

Sizes default to the Llama-3.1-8B shape.  With ``--reps 2`` a run is short enough to
sit under a profiler.
"""
from __future__ import annotations

import argparse
import math
import sys

import torch

from .csrc import ops
from .parts.attention import decode_splits

L2_BYTES = 126e6


def _time(fn, reps: int) -> float:
    """Mean microseconds of fn(i) over reps calls, after 3 warm-up calls."""
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    a.record()
    for i in range(reps):
        fn(i)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps * 1e3


def gemm_small_m(args) -> None:
    H, I, V = args.hidden, args.intermediate, args.vocab
    qkv = (args.heads + 2 * args.kv_heads) * args.head_dim
    shapes = [("qkv", qkv, H, False), ("o", H, args.heads * args.head_dim, False),
              ("gate_up+silu", I, H, True), ("down", H, I, False), ("head", V, H, False)]
    M = args.tokens
    for name, N, K, gated in shapes:
        rows = 2 * N if gated else N
        nbytes = rows * K * 2
        copies = max(2, int(3 * L2_BYTES // nbytes) + 1)          # walk through > 3 x L2 of weights
        ws = [torch.randn(rows, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        lib_out = torch.empty(M, rows, device="cuda", dtype=torch.bfloat16)
        if M <= ops.SMALL_M:
            kern = "gemm_small_m"
            own = _time(lambda i: ops.gemm_small_m(x, ws[i % copies], out, gated=gated), args.reps)
        else:
            kern = "gemm_mid_m"
            own = _time(lambda i: ops.gemm_mid_m(x, ws[i % copies], out, gated=gated), args.reps)
            ops.check_tc_status("cuda")
        lib = _time(lambda i: torch.mm(x, ws[i % copies].t(), out=lib_out), args.reps)
        print(f"{kern} {name:13s} M={M:2d} N={N:6d} K={K:5d}: {own:7.1f} us {nbytes / own / 1e6:5.2f} TB/s"
              f"   (vendor library: {lib:7.1f} us {nbytes / lib / 1e6:5.2f} TB/s)", flush=True)
        del ws


def gemm_tc(args) -> None:
    H, I, V = args.hidden, args.intermediate, args.vocab
    qkv = (args.heads + 2 * args.kv_heads) * args.head_dim
    shapes = [("qkv", qkv, H, False), ("o", H, args.heads * args.head_dim, False),
              ("gate_up+silu", I, H, True), ("down", H, I, False)]
    M = args.tokens
    for name, N, K, gated in shapes:
        rows = 2 * N if gated else N
        flops = 2.0 * M * rows * K
        copies = max(2, int(3 * L2_BYTES // (rows * K * 2)) + 1)
        ws = [torch.randn(rows, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        lib_out = torch.empty(M, rows, device="cuda", dtype=torch.bfloat16)
        own = _time(lambda i: ops.gemm_tc(x, ws[i % copies], out, gated=gated), args.reps)
        two = _time(lambda i: ops.gemm_tc(x, ws[i % copies], out, gated=gated, pair=True), args.reps)
        ops.check_tc_status("cuda")
        lib = _time(lambda i: torch.mm(x, ws[i % copies].t(), out=lib_out), args.reps)
        print(f"gemm_tc {name:13s} M={M:4d} N={N:6d} K={K:5d}: one CTA per tile {own:7.1f} us {flops / own / 1e6:7.1f} TFLOP/s,"
              f" CTA pairs {two:7.1f} us {flops / two / 1e6:7.1f} TFLOP/s"
              f"   (vendor library: {lib:7.1f} us {flops / lib / 1e6:7.1f} TFLOP/s)", flush=True)
        del ws


def _cache(args, n_seqs: int, ctx: int):
    page, nkv, d = args.page_size, args.kv_heads, args.head_dim
    per_seq = -(-ctx // page)
    pages = n_seqs * per_seq
    kc = torch.randn(pages, nkv, page, d, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn(pages, nkv, page, d, device="cuda", dtype=torch.bfloat16)
    tables = torch.randperm(pages, dtype=torch.int32).view(n_seqs, per_seq).cuda()
    return kc, vc, tables, per_seq


def attn_decode(args) -> None:
    nh, nkv, d, page, B, ctx = args.heads, args.kv_heads, args.head_dim, args.page_size, args.batch, args.context
    seq_bytes = ctx * nkv * d * 2 * 2
    n_seqs = max(B, int(3 * L2_BYTES // seq_bytes) // B * B + B)    # rotate through > 3 x L2 of cache
    kc, vc, tables, stride = _cache(args, n_seqs, ctx)
    q = torch.randn(B, (nh + 2 * nkv) * d, device="cuda", dtype=torch.bfloat16)
    cu = torch.arange(B + 1, dtype=torch.int32, device="cuda")
    ctxs = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    dec = torch.arange(B, dtype=torch.int32, device="cuda")
    out = torch.empty(B, nh * d, device="cuda", dtype=torch.bfloat16)
    bts = [tables[i:i + B].contiguous() for i in range(0, n_seqs, B)]
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    cap = [0] + [ops.attn_decode_cluster_capacity(torch.bfloat16, d, s, nh // nkv) for s in range(1, ops.ATTN_MAX_CLUSTER + 1)]
    print("clusters of s slices held at once:", cap[1:])
    splits = args.splits or decode_splits(B, nkv * -(-(nh // nkv) // 16), sms, cap)
    po = torch.empty(B * nh * splits * d, device="cuda")
    pm = torch.empty(B * nh * splits * 2, device="cuda")
    t = _time(lambda i: ops.attn_decode(q, q.shape[1], kc, vc, bts[i % len(bts)], stride, cu, ctxs, dec, B,
                                        splits, po, pm, out, nh, nkv, d, page, 0, 1 / math.sqrt(d)), args.reps)
    print(f"attn_decode+merge B={B} context={ctx} heads={nh}/{nkv} d={d} splits={splits}: {t:7.1f} us "
          f"{B * seq_bytes / t / 1e6:5.2f} TB/s of cache", flush=True)
    pieces = ops.attn_decode_flat_pieces(B, nh, nkv, d)
    po = torch.empty(pieces * 16 * d, device="cuda")
    pm = torch.empty(pieces * 16 * 2, device="cuda")
    prefix = torch.empty(ops.attn_decode_flat_prefix_ints(B, nh, nkv), dtype=torch.int32, device="cuda")
    t = _time(lambda i: ops.attn_decode_flat(q, q.shape[1], kc, vc, bts[i % len(bts)], stride, cu, ctxs, dec, B,
                                             po, pm, prefix, out, nh, nkv, d, page, 0, 1 / math.sqrt(d)), args.reps)
    print(f"attn_decode_flat (equal ranges of tiles) B={B} context={ctx}: {t:7.1f} us "
          f"{B * seq_bytes / t / 1e6:5.2f} TB/s of cache", flush=True)


def attn_prefill(args) -> None:
    nh, nkv, d, page, T = args.heads, args.kv_heads, args.head_dim, args.page_size, args.tokens
    kc, vc, tables, stride = _cache(args, 4, T)
    q = torch.randn(T, (nh + 2 * nkv) * d, device="cuda", dtype=torch.bfloat16)
    cu = torch.tensor([0, T], dtype=torch.int32, device="cuda")
    ctxs = torch.tensor([T], dtype=torch.int32, device="cuda")
    t16 = torch.arange(0, T, 16, dtype=torch.int32, device="cuda")
    t64 = torch.arange(0, T, 64, dtype=torch.int32, device="cuda")
    t128 = torch.arange(0, T, 128, dtype=torch.int32, device="cuda").flip(0).contiguous()   # longest first
    out = torch.empty(T, nh * d, device="cuda", dtype=torch.bfloat16)
    flops = 2.0 * 2.0 * nh * d * T * T / 2
    for name, tc in (("tcgen05, best for the shape", 1), ("tcgen05, two heads per CTA, steps of 64 keys", 3),
                     ("tcgen05, one head per CTA", 2), ("mma.sync", 0)):
        if tc and d not in (64, 128):
            continue
        t = _time(lambda i: ops.attn_prefill(q, q.shape[1], kc, vc, tables[i % 4:i % 4 + 1].contiguous(), stride, cu,
                                             ctxs, torch.zeros_like(t16), t16, len(t16), out, nh, nkv, d, page, 0,
                                             1 / math.sqrt(d), torch.zeros_like(t64), t64, len(t64),
                                             tile128_seq=torch.zeros_like(t128), tile128_q0=t128,
                                             num_tiles128=len(t128), allow_tc=tc), args.reps)
        if tc:
            ops.check_tc_status("cuda")
        print(f"attn_prefill ({name}) T={T} heads={nh}/{nkv} d={d}: {t:7.1f} us {flops / t / 1e6:6.1f} TFLOP/s (causal)",
              flush=True)


def sample(args) -> None:
    """Token selection from float32 logits [batch, vocab]: arg-max, then sampling with a
    temperature alone, with top-k, with top-p and with both."""
    B, V = args.batch, args.vocab
    torch.manual_seed(0)
    logits = torch.randn(B, V, device="cuda") * 3
    out = torch.empty(B, dtype=torch.int32, device="cuda")
    temp = torch.full((B,), 0.8, device="cuda")
    top_k = torch.full((B,), 50, dtype=torch.int32, device="cuda")
    top_p = torch.full((B,), 0.9, device="cuda")
    seeds = torch.arange(B, dtype=torch.int64, device="cuda")
    draw = torch.zeros(B, dtype=torch.int64, device="cuda")
    print(f"argmax rows={B} vocab={V}: {_time(lambda i: ops.argmax(logits, out), args.reps):7.1f} us", flush=True)
    for name, k, p in (("temperature only", None, None), ("top-k 50", top_k, None), ("top-p 0.9", None, top_p),
                       ("top-k 50 + top-p 0.9", top_k, top_p)):
        t = _time(lambda i: ops.sample(logits, temp, k, p, seeds, draw, out), args.reps)
        print(f"sample ({name}) rows={B} vocab={V}: {t:7.1f} us", flush=True)


def step_timeline(args) -> None:
    """Kernel timeline of one step of the whole model through CUPTI (torch.profiler): per kernel
    name the launches of the step, their summed durations and the idle time before them.  A
    decode step of --batch sequences at --context tokens (a captured graph for the batches the
    engine captures), or with --tokens a prompt step of that many tokens.  With programmatic
    dependent launch a kernel's duration includes the time it waits for the one before, so the
    durations of neighbours overlap; the step's total is the span from first start to last end."""
    import collections
    import json
    import os
    import time
    from torch.profiler import ProfilerActivity, profile
    from . import Engine, EngineConfig
    from .engine.batch import StepEntry
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "bench_shapes", args.shape + ".json")) as f:
        cfg = json.load(f)
    B, C, T = args.batch, args.context, args.prompt_tokens
    room = (C + 256) if not T else T + 64
    ecfg = EngineConfig(dtype="bfloat16", block_size=args.page_size,
                        num_blocks=(B + 1) * (-(-room // args.page_size)) + 64, max_batch_size=max(B, 8),
                        max_token_budget=max(2048, T) + B, prefill_chunk_size=max(2048, T),
                        max_model_len=max(room, 2048) + 64, max_queue_depth=0)
    eng = Engine(config=cfg, weights_seed=0, engine_config=ecfg)
    runner = eng.runner
    gen = torch.Generator().manual_seed(1)
    V = cfg["vocab_size"]
    rp = lambda k: torch.randint(0, V, (k,), generator=gen).tolist()
    if T:
        def one(i=[0]):
            i[0] += 1
            rid = f"p{i[0]}"
            runner.step([StepEntry(rid, rp(T), [T - 1])])
            runner.release(rid)
    else:
        ids = [f"d{j}" for j in range(B)]
        for rid in ids:
            for c0 in range(0, C, 2048):
                runner.step([StepEntry(rid, rp(min(2048, C - c0)), [])])
        toks = rp(B)
        out = torch.empty(B, dtype=torch.int32, device=runner.device)

        def one():
            ops.argmax(runner.step([StepEntry(rid, [toks[j]], [0]) for j, rid in enumerate(ids)]), out)
    for _ in range(6):
        one()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        one()
        torch.cuda.synchronize()
    ks = sorted(((e.time_range.start, e.time_range.end, e.name) for e in prof.events()
                 if "cuda" in str(e.device_type).lower()), key=lambda k: k[0])
    t0, prev = ks[0][0], ks[0][0]
    agg = collections.OrderedDict()
    for s0, e0, name in ks:
        a = agg.setdefault(name[:72], [0, 0.0, 0.0, 0.0])       # launches, duration, idle before, time to the end before
        a[0] += 1
        a[1] += e0 - s0
        a[2] += max(0.0, s0 - prev)
        a[3] += max(0.0, e0 - max(prev, s0)) if e0 > prev else 0.0
        prev = max(prev, e0)
    what = f"prompt step of {T} tokens" if T else f"decode step, batch {B}, context {C}"
    print(f"{args.shape}: {what}: {len(ks)} launches, {(ks[-1][1] - t0) / 1e3:.3f} ms from first start to last end")
    print("launches  duration us (each)   end-to-end us (each)   idle before us   kernel")
    for name, (n, d, g, eff) in sorted(agg.items(), key=lambda kv: -kv[1][3]):
        print(f"{n:8d}  {d:9.1f} ({d / n:6.1f})   {eff:9.1f} ({eff / n:6.1f})   {g:8.1f}   {name}")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m gollmgo_b200.microbench")
    ap.add_argument("kernel", choices=["gemm_small_m", "gemm_tc", "attn_decode", "attn_prefill", "sample", "step_timeline"])
    ap.add_argument("--tokens", type=int, default=None)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--reps", type=int, default=40)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--intermediate", type=int, default=14336)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--shape", default="llama_3_1_8b", help="step_timeline: a file of bench_shapes/")
    ap.add_argument("--prompt-tokens", type=int, default=0, help="step_timeline: a prompt step of so many tokens instead of a decode step")
    args = ap.parse_args(argv)
    if args.tokens is None:
        args.tokens = 8 if args.kernel == "gemm_small_m" else 2048
    {"gemm_small_m": gemm_small_m, "gemm_tc": gemm_tc, "attn_decode": attn_decode, "attn_prefill": attn_prefill,
     "sample": sample, "step_timeline": step_timeline}[args.kernel](args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
