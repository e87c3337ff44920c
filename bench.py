"""Benchmark of the engine's headline metric: decode tokens per second, Llama-3.1-8B
shape, bfloat16, random weights, batch 8 at a 2,048-token context (plus prefill of
2,048 tokens and decode at batch 1 and 64).  Prints ONE JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]

A "step" is one decode step.  ``value`` times K steps of the runner (graph replay
and on-device arg-max) with CUDA events; ``e2e`` times the same through the
Python entry point (Engine.step: host token ids in through pinned memory, sampled
tokens back to the host every step).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

with open(os.path.join(ROOT, "gollmgo_b200", "bench_shapes", "llama_3_1_8b.json")) as _f:
    LLAMA_3_1_8B = json.load(_f)      # the layer sizes of the headline configuration
CONTEXT = 2048          # every sequence starts decoding at this context
PREFILL_TOKENS = 2048
PAGE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    except (OSError, KeyError, ValueError):
        return {**FALLBACK_PEAKS, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, device=0):
        self.rows, self.proc, self.device = [], None, device

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.device}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = max(mx, float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def layer_weight_bytes(c, L):
    H, I, d = c["hidden_size"], c["intermediate_size"], c["head_dim"]
    nh, nkv = c["num_attention_heads"], c["num_key_value_heads"]
    per_layer = (nh + 2 * nkv) * d * H + nh * d * H + 3 * H * I + 2 * H
    return 2 * (L * per_layer + H + c["vocab_size"] * H)         # bf16; + final norm + LM head


def kv_bytes(c, L, contexts):
    return sum(2 * ctx * c["num_key_value_heads"] * c["head_dim"] * 2 * L for ctx in contexts)


def prefill_flops(c, L, T):
    H, I, d = c["hidden_size"], c["intermediate_size"], c["head_dim"]
    nh, nkv = c["num_attention_heads"], c["num_key_value_heads"]
    per_layer = (nh + 2 * nkv) * d * H + nh * d * H + 3 * H * I
    return 2.0 * T * L * per_layer + L * 2.0 * 2.0 * nh * d * T * T / 2 + 2.0 * H * c["vocab_size"]


def reference_arm(args) -> int:
    """The same metric on the reference: its five CUDA files built as they are and driven
    through their C API (baseline/reference_arm.py; nothing of gollmgo_b200 is imported)."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm as ra
    if args.gpus != 1:
        print(json.dumps({"impl": "reference", "unavailable": "the reference's engine runs on one GPU"}))
        return 0
    W, K, B = max(args.warmup, 3), max(args.steps, 1), args.batch
    cfg = dict(LLAMA_3_1_8B)
    L_full = cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = L = args.layers or L_full
    try:
        r = ra.run_bench(cfg, B, CONTEXT, K, W, PREFILL_TOKENS, points=() if args.skip_points else (1, 64),
                         clock_sampler=ClockSampler)
    except ra.Unavailable as exc:
        print(json.dumps({"impl": "reference", "unavailable": str(exc).replace("\n", " ")[:400]}))
        return 0
    pk = peaks()
    ms = r["ms_per_step"]
    ctx_mean = CONTEXT + W + (K + 1) / 2
    bytes_step = layer_weight_bytes(cfg, L) + kv_bytes(cfg, L, [ctx_mean] * B)
    achieved = bytes_step / (ms / 1e3) / 1e9
    pf_ms = r["prefill_ms"]
    line = {
        "metric": "decode tokens/s (Llama-3.1-8B shape, batch %d, context %d)" % (B, CONTEXT),
        "value": round(B / (ms / 1e3), 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids)", "impl": "reference",
        "config": {"model": "Llama-3.1-8B shape", "layers": L, "layers_of_configuration": L_full,
                   "hidden_size": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate_size": cfg["intermediate_size"], "vocab_size": cfg["vocab_size"],
                   "global_batch": B, "seq_len": CONTEXT, "context_start": CONTEXT, "decode_steps": K,
                   "parallelism": "single GPU", "max_seq_len": r["max_seq_len"],
                   "api": "gollmgo_model_forward_prefill + gollmgo_model_forward_paged (C API, ctypes)",
                   "l2": "inputs larger than L2 (weights 15 GB per step)", "peaks": pk["source"]},
        "e2e": {"value": round(B / r["wall_per_step"], 1), "unit": "tokens/s",
                "h2d_bytes_per_step": r["h2d_bytes_per_step"], "d2h_bytes_per_step": r["d2h_bytes_per_step"]},
        "clocks": r["clocks"],
        "prefill": {"value": round(PREFILL_TOKENS / (pf_ms / 1e3), 1), "tokens": PREFILL_TOKENS,
                    "ms": round(pf_ms, 3),
                    "frac": round(prefill_flops(cfg, L, PREFILL_TOKENS) / (pf_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": r["points"],
    }
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--skip-points", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(json.dumps({"error": "this engine runs on one GPU; --gpus must be 1", "n_gpus": args.gpus}))
        return 2
    W = max(args.warmup, 3)
    K = max(args.steps, 1)

    import torch
    from gollmgo_b200 import Engine, EngineConfig, SamplingParams
    from gollmgo_b200.csrc import ops
    from gollmgo_b200.engine.batch import StepEntry

    cfg = dict(LLAMA_3_1_8B)
    L_full = cfg["num_hidden_layers"]
    L = args.layers or L_full
    cfg["num_hidden_layers"] = L
    B = args.batch
    batches = sorted({B} | (set() if args.skip_points else {1, 64}))
    gen_room = K + W + 8
    tokens_per_seq = CONTEXT + 2 * gen_room + 64
    max_b = max(batches)
    ecfg = EngineConfig(dtype="bfloat16", block_size=PAGE,
                        num_blocks=(max_b + 1) * (-(-tokens_per_seq // PAGE)) + 256,
                        max_batch_size=max(max_b, 8), max_token_budget=PREFILL_TOKENS + max_b,
                        prefill_chunk_size=PREFILL_TOKENS, max_model_len=tokens_per_seq + PREFILL_TOKENS,
                        max_queue_depth=0)
    eng = Engine(config=cfg, weights_seed=0, engine_config=ecfg)
    runner = eng.runner
    dev = runner.device
    gen = torch.Generator().manual_seed(1)
    V = cfg["vocab_size"]
    rand_prompt = lambda n: torch.randint(0, V, (n,), generator=gen).tolist()
    pk = peaks()

    def timed(fn, n):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(dev)
        a.record()
        for i in range(n):
            fn(i)
        b.record()
        torch.cuda.synchronize(dev)
        return a.elapsed_time(b)

    # ---- prefill of 2,048 tokens in one step (host token lists made before the timed steps)
    reps = 8
    pf_prompts = [rand_prompt(PREFILL_TOKENS) for _ in range(reps)]

    def prefill_once(i):
        rid = f"pf{i}-{time.monotonic_ns()}"
        runner.step([StepEntry(rid, pf_prompts[i % reps], [PREFILL_TOKENS - 1])])
        runner.release(rid)
    for i in range(3):
        prefill_once(i)
    pf_ms = timed(prefill_once, reps) / reps
    pf_flops = prefill_flops(cfg, L, PREFILL_TOKENS)
    prefill = {"value": round(PREFILL_TOKENS / (pf_ms / 1e3), 1), "tokens": PREFILL_TOKENS,
               "ms": round(pf_ms, 3), "frac": round(pf_flops / (pf_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}

    # ---- decode at each batch size: sequences prefilled to CONTEXT, then W + K single-token steps
    argmax_out = torch.empty(max_b, dtype=torch.int32, device=dev)

    def decode_run(b, steps, warm, sample_clocks=False):
        ids = [f"d{b}-{j}" for j in range(b)]
        for rid in ids:
            runner.step([StepEntry(rid, rand_prompt(CONTEXT), [])])
        toks = rand_prompt(b)

        def one(i):
            logits = runner.step([StepEntry(rid, [toks[j]], [0]) for j, rid in enumerate(ids)])
            ops.argmax(logits, argmax_out[:b])
        for i in range(warm):
            one(i)
        clocks = ClockSampler(dev.index or 0) if sample_clocks else None
        l0 = ops.launches
        if clocks:
            clocks.start()
        ms = timed(one, steps)
        launches = ops.launches - l0
        c = clocks.stop() if clocks else None
        ctx_mean = CONTEXT + warm + (steps + 1) / 2
        for rid in ids:
            runner.release(rid)
        return ms / steps, launches, c, ctx_mean

    results = {}
    for b in batches:
        results[b] = decode_run(b, K, W, sample_clocks=(b == B))
    ms_step, launches, clocks, ctx_mean = results[B]
    bytes_step = layer_weight_bytes(cfg, L) + kv_bytes(cfg, L, [ctx_mean] * B)
    achieved = bytes_step / (ms_step / 1e3) / 1e9
    value = B / (ms_step / 1e3)

    # ---- end to end through the Python entry point: host tokens in, sampled tokens out, every step
    # no sequence ends inside the timed steps (the first ones decode while the last prompts are still read)
    params = SamplingParams(max_tokens=W + K + 64, ignore_eos=True)
    for j in range(B):
        eng.enqueue(rand_prompt(CONTEXT), params)
    while any(s.state.value != "DECODING" for s in eng.scheduler.running.values()) or eng.scheduler.waiting:
        eng.step()
    for _ in range(W):
        eng.step()
    torch.cuda.synchronize(dev)
    t0 = time.perf_counter()
    n_tok = 0
    for _ in range(K):
        n_tok += len(eng.step())
    torch.cuda.synchronize(dev)
    e2e_s = time.perf_counter() - t0
    # bytes of the step's packed metadata (token ids, positions, block tables, ...) that go to the device
    metas = sorted((k[0] if isinstance(k, tuple) else k, c.meta.numel() * 4) for k, c in runner._graphs.items())
    lay = next((nbytes for bucket, nbytes in metas if bucket >= B), 0)
    eng.stop()
    e2e = {"value": round(n_tok / e2e_s, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(lay),
           "d2h_bytes_per_step": 4 * B}

    line = {
        "metric": "decode tokens/s (Llama-3.1-8B shape, batch %d, context %d)" % (B, CONTEXT),
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids)",
        "impl": "ours",
        "config": {"model": "Llama-3.1-8B shape", "layers": L, "layers_of_configuration": L_full,
                   "hidden_size": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate_size": cfg["intermediate_size"], "vocab_size": V,
                   "global_batch": B, "seq_len": CONTEXT, "context_start": CONTEXT,
                   "decode_steps": K, "page_size": PAGE, "parallelism": "single GPU",
                   "cuda_graphs": True, "l2": "inputs larger than L2 (weights 15 GB per step)",
                   "peaks": pk["source"]},
        "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": {f"decode_b{b}": round(b / (results[b][0] / 1e3), 1) for b in batches if b != B},
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
