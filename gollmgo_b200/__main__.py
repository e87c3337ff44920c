"""Command line: ``python -m gollmgo_b200 generate | bench | doctor``.

Option names and meanings are the reference's where it has them
(cmd/gollmgo/main.go:52-60 serve flags --config --model --device --log-level;
:227-240 bench flags --mode --num-prompts --prompt-len --output-len
--warmup-requests --repetitions --model --config; :591-632 doctor).  The engine
keys of --config are those of its server config (internal/config/config.go:33-78).
``serve`` (the HTTP server) is not part of this engine.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import subprocess
import sys
import time


def _engine_flags(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("--model", default="", help="local model folder (config.json + *.safetensors)")
    ap.add_argument("--config", default="", help="JSON file with engine keys: max_batch_size, "
                    "max_token_budget, max_queue_depth, prefill_chunk_size, block_size, max_memory_fraction")
    ap.add_argument("--device", type=int, default=0, help="CUDA device index")
    ap.add_argument("--log-level", default="info", choices=["debug", "info", "warn", "error"])
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--random-weights", default="", metavar="CONFIG_JSON",
                    help="a config.json to run with random weights instead of --model")
    ap.add_argument("--seed", type=int, default=0, help="seed of the random weights")
    ap.add_argument("--max-batch-size", type=int)
    ap.add_argument("--max-token-budget", type=int)
    ap.add_argument("--max-queue-depth", type=int)
    ap.add_argument("--prefill-chunk-size", type=int)
    ap.add_argument("--block-size", type=int)
    ap.add_argument("--num-blocks", type=int, help="cache pages (default: from --max-memory-fraction)")
    ap.add_argument("--max-memory-fraction", type=float)
    ap.add_argument("--max-model-len", type=int)
    ap.add_argument("--no-cuda-graphs", action="store_true")


def _log(args, level: str, msg: str, **kv) -> None:
    order = ["debug", "info", "warn", "error"]
    if order.index(level) >= order.index(args.log_level):
        extra = " ".join(f"{k}={v}" for k, v in kv.items())
        print(f"time={datetime.datetime.now().isoformat(timespec='seconds')} level={level.upper()} "
              f"msg=\"{msg}\" {extra}".rstrip(), file=sys.stderr, flush=True)


def _make_engine(args):
    from .config import EngineConfig
    from .engine.llm_engine import Engine
    ecfg = EngineConfig(dtype=args.dtype, device=args.device, cuda_graphs=not args.no_cuda_graphs)
    if args.config:
        with open(args.config) as f:
            data = json.load(f)
        data = {**data, **data.get("server", {})}       # reference: internal/config/load.go:21-30
        for k in ("max_batch_size", "max_token_budget", "max_queue_depth", "prefill_chunk_size",
                  "block_size", "max_memory_fraction"):
            if k in data:
                setattr(ecfg, k, data[k])
    for k in ("max_batch_size", "max_token_budget", "max_queue_depth", "prefill_chunk_size",
              "block_size", "num_blocks", "max_memory_fraction", "max_model_len"):
        v = getattr(args, k)
        if v is not None:
            setattr(ecfg, k, v)
    t0 = time.time()
    if args.random_weights:
        with open(args.random_weights) as f:
            cfg = json.load(f)
        eng = Engine(config=cfg, weights_seed=args.seed, engine_config=ecfg)
    elif args.model:
        eng = Engine(args.model, engine_config=ecfg)
    else:
        raise SystemExit("error: give --model DIR or --random-weights CONFIG_JSON")
    rep = eng.runner.memory_report()
    _log(args, "info", "engine ready", seconds=f"{time.time() - t0:.1f}", dtype=args.dtype,
         weights_gb=f"{rep['weights_bytes'] / 1e9:.2f}", cache_pages=rep["cache_pages"],
         page_size=rep["page_size"])
    return eng


def cmd_generate(argv) -> int:
    ap = argparse.ArgumentParser(prog="gollmgo_b200 generate")
    _engine_flags(ap)
    ap.add_argument("--prompt-ids", action="append", default=[],
                    help="comma-separated token ids; may be given several times")
    ap.add_argument("--prompt-len", type=int, default=0, help="instead: a synthetic prompt of this length")
    ap.add_argument("--num-prompts", type=int, default=1)
    ap.add_argument("--max-tokens", type=int, default=256)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=0.0)
    ap.add_argument("--sampling-seed", type=int, default=None)
    ap.add_argument("--ignore-eos", action="store_true")
    args = ap.parse_args(argv)
    from .sampling import SamplingParams
    eng = _make_engine(args)
    V = eng.spec.vocab_size
    prompts = [[int(t) for t in p.split(",") if t.strip()] for p in args.prompt_ids]
    if not prompts:
        n = args.prompt_len or 8
        prompts = [[(j + i) % min(V, 255) for j in range(n)] for i in range(args.num_prompts)]
    params = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                            seed=args.sampling_seed, max_tokens=args.max_tokens,
                            ignore_eos=args.ignore_eos)
    outs = eng.generate(prompts, params)
    for o in outs:
        print(json.dumps({"request_id": o.request_id, "prompt_token_ids": o.prompt_token_ids,
                          "token_ids": o.token_ids, "finish_reason": o.finish_reason}))
    return 0


def _percentile(xs, q):
    if not xs:
        return 0.0
    xs = sorted(xs)
    k = (len(xs) - 1) * q
    lo, hi = int(k), min(int(k) + 1, len(xs) - 1)
    return xs[lo] + (xs[hi] - xs[lo]) * (k - lo)


def _git_sha() -> str:
    try:
        return subprocess.run(["git", "rev-parse", "--short", "HEAD"], capture_output=True, text=True,
                              cwd=os.path.dirname(os.path.abspath(__file__))).stdout.strip() or "unknown"
    except OSError:
        return "unknown"


def cmd_bench(argv) -> int:
    ap = argparse.ArgumentParser(prog="gollmgo_b200 bench")
    _engine_flags(ap)
    ap.add_argument("--mode", default="offline", choices=["offline", "synthetic", "decode", "prefill"],
                    help="offline/synthetic: synthetic token prompts through the engine; decode: --batch "
                         "sequences at --context tokens, --output-len single-token steps, timed on the "
                         "device; prefill: one prompt of --prompt-len tokens in one step "
                         "(the reference's serving mode needs its HTTP server and is not built)")
    ap.add_argument("--batch", type=int, default=8, help="sequences (decode mode)")
    ap.add_argument("--context", type=int, default=2048, help="tokens cached per sequence (decode mode)")
    ap.add_argument("--num-prompts", type=int, default=100)
    ap.add_argument("--prompt-len", type=int, default=128)
    ap.add_argument("--output-len", type=int, default=128)
    ap.add_argument("--warmup-requests", type=int, default=0)
    ap.add_argument("--repetitions", type=int, default=1)
    ap.add_argument("--concurrency", type=int, default=0,
                    help="closed loop with this many requests in the engine at a time, the next handed in "
                         "when one finishes (the reference's serving benchmark: 4); 0: all prompts at once")
    ap.add_argument("--prompt-len-range", default="", metavar="LO,HI",
                    help="prompt lengths drawn uniformly from [LO, HI] (from --workload-seed) instead of --prompt-len")
    ap.add_argument("--output-len-range", default="", metavar="LO,HI",
                    help="output lengths drawn uniformly from [LO, HI] instead of --output-len")
    ap.add_argument("--workload-seed", type=int, default=0, help="seed of the drawn lengths and token ids")
    args = ap.parse_args(argv)
    import random
    import torch
    from .sampling import SamplingParams
    if args.mode in ("decode", "prefill"):
        return _bench_step(args)

    def span(text, what):
        try:
            lo, hi = (int(x) for x in text.split(","))
        except ValueError:
            raise SystemExit(f"error: {what} wants LO,HI (two integers), got {text!r}") from None
        if not (1 <= lo <= hi):
            raise SystemExit(f"error: {what} needs 1 <= LO <= HI, got {text!r}")
        return lo, hi
    p_span = span(args.prompt_len_range, "--prompt-len-range") if args.prompt_len_range else None
    o_span = span(args.output_len_range, "--output-len-range") if args.output_len_range else None
    eng = _make_engine(args)
    V = eng.spec.vocab_size

    def workload(n, seed):
        """n (prompt, params).  Fixed lengths: prompts as the reference's offline bench makes
        them, prompt[j] = (j + i) % 255 (cmd/gollmgo/main.go:335-422).  Drawn lengths: lengths
        and token ids uniform from the seed."""
        rng = random.Random(seed)
        out = []
        for i in range(n):
            plen = rng.randint(*p_span) if p_span else args.prompt_len
            olen = rng.randint(*o_span) if o_span else args.output_len
            if p_span or o_span:
                prompt = [rng.randrange(V) for _ in range(plen)]
            else:
                prompt = [(j + i + seed) % min(V, 255) for j in range(plen)]
            out.append((prompt, SamplingParams(max_tokens=olen, ignore_eos=True)))
        return out

    def run(items):
        return eng.generate([p for p, _ in items], [q for _, q in items], concurrency=args.concurrency)
    if args.warmup_requests:
        run(workload(args.warmup_requests, args.workload_seed + 7))
    result = None
    for rep in range(args.repetitions):
        items = workload(args.num_prompts, args.workload_seed)
        s0 = (eng.stats.steps, eng.stats.batch_sum, eng.stats.preemptions, eng.stats.prefill_tokens,
              eng.stats.decode_tokens)
        for g in eng.runner.cache.groups:
            g.pool.high_water = g.pool.num_used
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = run(items)
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - t0
        toks = sum(len(o.token_ids) for o in outs)
        steps = eng.stats.steps - s0[0]
        itl = [b - a for o in outs for a, b in zip(o.token_times, o.token_times[1:])]
        ttft = [o.ttft_s for o in outs if o.ttft_s is not None]
        e2e = [o.e2e_s for o in outs if o.e2e_s is not None]
        ms = lambda xs, q: round(_percentile(xs, q) * 1e3, 3)
        result = {
            "timestamp": datetime.datetime.now(datetime.timezone.utc).isoformat(timespec="seconds"),
            "git_sha": _git_sha(), "hardware": torch.cuda.get_device_name(args.device),
            "mode": args.mode, "num_prompts": args.num_prompts, "measured_requests": len(outs),
            "prompt_len": args.prompt_len if not p_span else None, "output_len": args.output_len if not o_span else None,
            "prompt_len_range": list(p_span) if p_span else None, "output_len_range": list(o_span) if o_span else None,
            "workload_seed": args.workload_seed,
            "prompt_tokens": sum(len(p) for p, _ in items), "output_tokens": toks,
            "warmup_requests": args.warmup_requests, "repetitions": args.repetitions,
            "concurrency": args.concurrency,
            "prompt_generation": "synthetic token ids", "token_count_mode": "exact",
            "elapsed_seconds": round(elapsed, 4), "tokens_per_second": round(toks / elapsed, 2),
            "total_tokens_per_second": round((toks + sum(len(p) for p, _ in items)) / elapsed, 2),
            "requests_per_second": round(len(outs) / elapsed, 3),
            "error_count": sum(1 for o in outs if o.finish_reason == "error"),
            "ttft_p50_ms": ms(ttft, .5), "ttft_p95_ms": ms(ttft, .95), "ttft_p99_ms": ms(ttft, .99),
            "e2e_p50_ms": ms(e2e, .5), "e2e_p95_ms": ms(e2e, .95), "e2e_p99_ms": ms(e2e, .99),
            "itl_p50_ms": ms(itl, .5), "itl_p95_ms": ms(itl, .95), "itl_p99_ms": ms(itl, .99),
            "dtype": args.dtype, "engine_steps": steps,
            "mean_batch": round((eng.stats.batch_sum - s0[1]) / max(steps, 1), 2),
            "mean_tokens_per_step": round((eng.stats.prefill_tokens - s0[3] + eng.stats.decode_tokens - s0[4])
                                          / max(steps, 1), 1),
            "preemptions": eng.stats.preemptions - s0[2],
            "pages_high_water": max((g.pool.high_water for g in eng.runner.cache.groups), default=0),
            "cache_pages": eng.runner.num_pages, "page_size": eng.runner.cache.page_size,
        }
        _log(args, "info", "repetition done", rep=rep, tokens_per_second=result["tokens_per_second"])
    print(json.dumps(result, indent=2))
    return 0


def _bench_step(args) -> int:
    """Device-timed single steps through the runner (no scheduler, no sampling on the host)."""
    import torch
    from .csrc import ops
    from .engine.batch import StepEntry
    if args.mode == "decode":
        need = args.batch * (args.context + args.output_len + 16)
        args.max_batch_size = max(args.max_batch_size or 0, args.batch)
        args.max_token_budget = max(args.max_token_budget or 0, args.context)
    else:
        need = 2 * args.prompt_len + 64
        args.max_token_budget = max(args.max_token_budget or 0, args.prompt_len)
    bs = args.block_size or 16
    args.num_blocks = args.num_blocks or (-(-need // bs) + 4 * (args.batch + 1))
    args.max_model_len = args.max_model_len or (args.context + args.output_len + args.prompt_len + 64)
    eng = _make_engine(args)
    runner, V = eng.runner, eng.spec.vocab_size
    gen = torch.Generator().manual_seed(args.seed)
    rand = lambda n: torch.randint(0, V, (n,), generator=gen).tolist()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.mode == "prefill":
        def once(i):
            runner.step([StepEntry(f"p{i}", rand(args.prompt_len), [args.prompt_len - 1])])
            runner.release(f"p{i}")
        for i in range(3):
            once(i)
        reps = max(args.repetitions, 3)
        torch.cuda.synchronize()
        a.record()
        for i in range(reps):
            once(3 + i)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / reps
        result = {"mode": "prefill", "prompt_len": args.prompt_len, "ms_per_step": round(ms, 3),
                  "tokens_per_second": round(args.prompt_len / ms * 1e3, 1)}
    else:
        ids = [f"d{j}" for j in range(args.batch)]
        for rid in ids:
            runner.step([StepEntry(rid, rand(args.context), [])])
        toks = rand(args.batch)
        out = torch.empty(args.batch, dtype=torch.int32, device=runner.device)

        def one():
            logits = runner.step([StepEntry(rid, [toks[j]], [0]) for j, rid in enumerate(ids)])
            ops.argmax(logits, out)
        warm = max(3, args.warmup_requests)
        steps = max(1, args.output_len - warm)
        for _ in range(warm):
            one()
        torch.cuda.synchronize()
        a.record()
        for _ in range(steps):
            one()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / steps
        result = {"mode": "decode", "batch": args.batch, "context": args.context, "steps": steps,
                  "ms_per_step": round(ms, 4), "tokens_per_second": round(args.batch / ms * 1e3, 1)}
    runner.check_kernels()
    result.update({"timestamp": datetime.datetime.now(datetime.timezone.utc).isoformat(timespec="seconds"),
                   "git_sha": _git_sha(), "hardware": torch.cuda.get_device_name(args.device),
                   "dtype": args.dtype, **runner.memory_report()})
    print(json.dumps(result, indent=2))
    return 0


def cmd_doctor(argv) -> int:
    ap = argparse.ArgumentParser(prog="gollmgo_b200 doctor")
    ap.add_argument("--device", type=int, default=0)
    args = ap.parse_args(argv)
    import shutil
    import torch
    ok = True

    def line(name, good, detail):
        nonlocal ok
        ok &= bool(good)
        print(f"[{'ok' if good else 'FAIL'}] {name}: {detail}")
    line("python", True, sys.version.split()[0])
    line("torch", True, torch.__version__)
    line("nvcc", shutil.which("nvcc") or os.path.exists("/usr/local/cuda/bin/nvcc"),
         shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc")
    has = torch.cuda.is_available()
    line("cuda device", has, torch.cuda.get_device_name(args.device) if has else "none visible")
    if has:
        p = torch.cuda.get_device_properties(args.device)
        line("compute capability", p.major >= 10, f"sm_{p.major}{p.minor}, {p.multi_processor_count} SMs, "
             f"{p.total_memory / 2**30:.0f} GiB")
        try:
            from .csrc import ops
            line("kernel library", True, ops.library_file())
        except Exception as e:  # noqa: BLE001
            line("kernel library", False, str(e))
    return 0 if ok else 1


def cmd_replay(argv) -> int:
    """Trace replay (the same as bin/trace_run): steps as JSON lines on standard input, logits at
    the wanted places to <out>/<step>.f32, `done <step>` after every step."""
    ap = argparse.ArgumentParser(prog="python -m gollmgo_b200 replay")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--no-cuda-graphs", action="store_true")
    args = ap.parse_args(argv)
    from .engine.trace import make_trace_runner, replay
    runner = make_trace_runner(args.model, args.dtype, args.max_tokens, args.block_size,
                               cuda_graphs=not args.no_cuda_graphs)
    replay(runner, sys.stdin, args.out)
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    cmds = {"generate": cmd_generate, "bench": cmd_bench, "doctor": cmd_doctor, "replay": cmd_replay}
    if not argv or argv[0] in ("-h", "--help") or argv[0] not in cmds:
        print("usage: python -m gollmgo_b200 <command> [flags]\n\ncommands:\n"
              "  generate  generate tokens for prompts given as token ids\n"
              "  bench     run synthetic prompts through the engine and print a result JSON\n"
              "  doctor    check the toolchain, the device and the kernel library\n"
              "  replay    feed given token ids step by step (JSON lines on stdin) and write logits\n",
              file=sys.stderr)
        return 0 if argv and argv[0] in ("-h", "--help") else 1
    return cmds[argv[0]](argv[1:])


if __name__ == "__main__":
    sys.exit(main())
