"""Generation through the Python entry point against the plain implementation:
greedy and seeded temperature sampling, the first tokens of a sequence, long
decoding over many pages, a pool so small that requests are preempted and
recomputed, and the command line."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_llama as P
import tiny_configs
import trace_tools as tt

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models(tmp_path_factory, cuda_device):
    tmp = str(tmp_path_factory.mktemp("models"))
    out = {}
    for name in ("tiny_a", "tiny_b"):
        cfg, page, std, jitter = tiny_configs.get(name)
        d = tt.model_folder(tmp, name, cfg, seed=21, std=std, jitter=jitter, dtype="float32")
        out[name] = (d, cfg, page, tt.load_weights(d))
    return out


def near_best(weights, cfg, prompt, tokens, slack):
    """Every token is (nearly) the plain implementation's best given the same history."""
    logits = P.forward(weights, cfg, prompt + tokens)
    for i, tok in enumerate(tokens):
        row = logits[len(prompt) - 1 + i]
        assert float(row.max() - row[tok]) <= slack * float(row.abs().max()), f"token {i} = {tok}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_workload_of_tiny_a(models, dtype):
    """Three requests with prompts of 7, 13 and 1 tokens, 8 greedy tokens each."""
    from gollmgo_b200 import Engine, SamplingParams
    d, cfg, page, w = models["tiny_a"]
    reqs = tt.random_requests(cfg["vocab_size"], [7, 13, 1], seed=1)
    eng = Engine(d, dtype=dtype, block_size=page, num_blocks=16, max_batch_size=4, max_token_budget=64)
    outs = eng.generate(list(reqs.values()), SamplingParams(max_tokens=8, ignore_eos=True))
    for prompt, o in zip(reqs.values(), outs):
        assert len(o.token_ids) == 8 and o.finish_reason == "length"
        if dtype == "float32":
            assert o.token_ids == P.generate(w, cfg, prompt, 8, cast=torch.float32)
        else:
            near_best(w, cfg, prompt, o.token_ids, 0.05)
    eng.runner.cache.audit()
    assert eng.runner.cache.free_pages() == 16


def test_temperature_workload_of_tiny_b_is_seeded_and_batch_independent(models):
    """Four requests (1, 5, 37, 70 tokens), prompts cut into portions of 16, 12 tokens each
    at temperature 0.8 with a seed: equal to the plain sampler, alone or in a batch."""
    from gollmgo_b200 import Engine, SamplingParams
    d, cfg, page, w = models["tiny_b"]
    reqs = list(tt.random_requests(cfg["vocab_size"], [1, 5, 37, 70], seed=2).values())
    params = [SamplingParams(temperature=0.8, seed=1000 + i, max_tokens=12, ignore_eos=True) for i in range(4)]
    eng = Engine(d, dtype="float32", block_size=page, num_blocks=64, max_batch_size=4,
                 max_token_budget=48, prefill_chunk_size=16)
    together = [o.token_ids for o in eng.generate(reqs, params)]
    alone = [eng.generate([r], [p])[0].token_ids for r, p in zip(reqs, params)]
    assert together == alone
    for prompt, p, got in zip(reqs, params, together):
        want = P.generate(w, cfg, prompt, 12, temperature=0.8, seed=p.seed, cast=torch.float32)
        assert got == want
    greedy = eng.generate(reqs, SamplingParams(max_tokens=12, ignore_eos=True))
    for prompt, o in zip(reqs, greedy):
        assert o.token_ids == P.generate(w, cfg, prompt, 12, cast=torch.float32)
    assert eng.runner.cache.free_pages() == 64


def test_temperature_top_k_top_p_in_bfloat16_follow_the_plain_sampler(models):
    """The bfloat16 engine with temperature, top-k and top-p at once.  Its logits are the plain
    ones up to rounding, so a draw that falls next to a border of the plain distribution may
    pick the neighbour: with the engine's own tokens as history, every token must be one the
    plain sampler could have drawn (among the plain top-k, with a slack of the rounding), most
    must be the very token the plain sampler draws from the same uniform number, and the same
    seeds give the same tokens again."""
    from gollmgo_b200 import Engine, SamplingParams
    d, cfg, page, w = models["tiny_b"]
    reqs = list(tt.random_requests(cfg["vocab_size"], [3, 21, 37, 70], seed=4).values())
    K, TOP_P, T, N = 12, 0.9, 0.7, 16
    params = [SamplingParams(temperature=T, top_k=K, top_p=TOP_P, seed=500 + i, max_tokens=N, ignore_eos=True)
              for i in range(4)]
    eng = Engine(d, dtype="bfloat16", block_size=page, num_blocks=64, max_batch_size=4,
                 max_token_budget=48, prefill_chunk_size=16)
    first = [o.token_ids for o in eng.generate(reqs, params)]
    again = [o.token_ids for o in eng.generate(reqs, params)]
    assert first == again
    same = total = 0
    for prompt, p, toks in zip(reqs, params, first):
        assert len(toks) == N
        logits = P.forward(w, cfg, prompt + toks)
        for n, tok in enumerate(toks):
            row = logits[len(prompt) - 1 + n].to(torch.float32)
            kth = torch.topk(row, K).values[-1]
            assert float(row[tok]) >= float(kth) - 4e-2 * float(row.abs().max()), f"token {n} = {tok} is no candidate"
            same += int(tok == P.sample(row, T, p.seed, n, K, TOP_P))
            total += 1
    assert same >= 0.75 * total, f"only {same} of {total} tokens are the plain sampler's"
    assert eng.runner.cache.free_pages() == 64


def test_eos_stops_and_is_delivered(models):
    from gollmgo_b200 import Engine, SamplingParams
    d, cfg, page, w = models["tiny_b"]
    prompt = [9, 8, 7]
    free_run = P.generate(w, cfg, prompt, 10, cast=torch.float32)
    cfg2 = dict(cfg, eos_token_id=[free_run[3]])
    d2 = os.path.join(os.path.dirname(d), "tiny_b_eos")
    os.makedirs(d2, exist_ok=True)
    os.link(os.path.join(d, "model.safetensors"), os.path.join(d2, "model.safetensors")) \
        if not os.path.exists(os.path.join(d2, "model.safetensors")) else None
    with open(os.path.join(d2, "config.json"), "w") as f:
        json.dump(cfg2, f)
    eng = Engine(d2, dtype="float32", block_size=page, num_blocks=16, max_batch_size=2, max_token_budget=32)
    o = eng.generate([prompt], SamplingParams(max_tokens=10))[0]
    stop = free_run.index(free_run[3])
    assert o.token_ids == free_run[:stop + 1] and o.finish_reason == "stop"
    o2 = eng.generate([prompt], SamplingParams(max_tokens=10, ignore_eos=True))[0]
    assert o2.token_ids == free_run and o2.finish_reason == "length"


def test_one_step_lookahead_drops_what_follows_an_end_token(models):
    """The engine launches a step before it has read the tokens of the step before.  A
    request that ends on an end-of-sequence token has then taken part in one step too
    many: that token is dropped, its neighbours are not disturbed, pages come back."""
    from gollmgo_b200 import Engine, SamplingParams
    d, cfg, page, w = models["tiny_a"]
    prompts = list(tt.random_requests(cfg["vocab_size"], [9, 4, 21, 2], seed=8).values())
    free = [P.generate(w, cfg, p, 14, cast=torch.float32) for p in prompts]
    eos = {free[0][5], free[2][9]}                 # request 0 ends at its 6th token, request 2 at its 10th
    want = [P.generate(w, cfg, p, 14, eos=eos, cast=torch.float32) for p in prompts]
    assert len(want[0]) <= 6 and len(want[2]) <= 10
    d2 = os.path.join(os.path.dirname(d), "tiny_a_eos")
    os.makedirs(d2, exist_ok=True)
    if not os.path.exists(os.path.join(d2, "model.safetensors")):
        os.link(os.path.join(d, "model.safetensors"), os.path.join(d2, "model.safetensors"))
    with open(os.path.join(d2, "config.json"), "w") as f:
        json.dump(dict(cfg, eos_token_id=sorted(eos)), f)
    eng = Engine(d2, dtype="float32", block_size=page, num_blocks=24, max_batch_size=4, max_token_budget=64)
    outs = eng.generate(prompts, SamplingParams(max_tokens=14))
    assert [o.token_ids for o in outs] == want
    assert [o.finish_reason for o in outs] == ["stop" if len(x) < 14 or x[-1] in eos else "length" for x in want]
    stream = []
    for p in prompts:
        eng.enqueue(p, SamplingParams(max_tokens=14))
    while eng.has_unfinished():
        stream.extend(eng.step())
    per_req = {}
    for r in stream:
        per_req.setdefault(r.request_id, []).append(r)
    assert [[r.token_id for r in v] for v in per_req.values()] == want
    assert all(v[-1].finished and not any(r.finished for r in v[:-1]) for v in per_req.values())
    eng.runner.cache.audit()
    assert eng.runner.cache.free_pages() == 24


@pytest.mark.parametrize("dtype,tol", [("float32", 1e-4), ("bfloat16", 6e-2)])
def test_first_tokens_and_long_decoding(models, dtype, tol):
    """Prompts of 1, 2 and 3 tokens, then 230 tokens decoded one by one through the
    runner (captured steps included), every logit row against the whole sequence."""
    from gollmgo_b200.config import EngineConfig
    from gollmgo_b200.engine.batch import StepEntry
    from gollmgo_b200.engine.runner import load_runner
    d, cfg, page, w = models["tiny_b"]
    runner = load_runner(d, EngineConfig(dtype=dtype, block_size=page, num_blocks=96, max_batch_size=4,
                                         max_token_budget=64, max_model_len=256))
    seqs = tt.random_requests(cfg["vocab_size"], [233, 234, 235], seed=3)
    refs = tt.plain_logits(w, cfg, seqs)
    names = list(seqs)
    first = {n: i + 1 for i, n in enumerate(names)}
    got = {n: [] for n in names}
    out = runner.step([StepEntry(n, seqs[n][:first[n]], range(first[n])) for n in names]).cpu().double()
    i = 0
    for n in names:
        got[n].append(out[i:i + first[n]])
        i += first[n]
    for t in range(1, 233):
        step = [n for n in names if first[n] + t - 1 < len(seqs[n])]
        out = runner.step([StepEntry(n, [seqs[n][first[n] + t - 1]], [0]) for n in step]).cpu().double()
        for j, n in enumerate(step):
            got[n].append(out[j:j + 1])
    for n in names:
        rows = torch.cat(got[n])
        ref = refs[n][:rows.shape[0]]
        err = ((rows - ref).abs().amax(dim=1) / ref.abs().amax(dim=1)).max()
        assert float(err) <= tol, f"{n}: worst relative error {float(err):.2e}"
        assert rows.shape[0] >= 230


@pytest.mark.parametrize("name", ["tiny_d", "tiny_e"])
def test_decode_kernel_for_large_batches_inside_the_engine(tmp_path, cuda_device, monkeypatch, name):
    """The decode attention that cuts all tiles into equal ranges is chosen when a step has more
    (token, kv head) pairs than CTAs fit at once; with the threshold lowered it runs for every
    decode step of a tiny model (head sizes 64 and 128, one with a window): every logit row of
    long decoding against the whole sequence, as with the sliced kernel."""
    import importlib
    A = importlib.import_module("gollmgo_b200.parts.attention")
    monkeypatch.setattr(A, "FLAT_DECODE_FILL", 1e-6)
    from gollmgo_b200.config import EngineConfig
    from gollmgo_b200.engine.batch import StepEntry
    from gollmgo_b200.engine.runner import load_runner
    cfg, page, std, jitter = tiny_configs.get(name)
    d = tt.model_folder(str(tmp_path), name, cfg, seed=31, std=std, jitter=jitter, dtype="bfloat16")
    w = tt.load_weights(d)
    runner = load_runner(d, EngineConfig(dtype="bfloat16", block_size=page, num_blocks=96, max_batch_size=4,
                                         max_token_budget=64, max_model_len=256))
    assert runner.model.blocks[0].mixer._flat_ok
    seqs = tt.random_requests(cfg["vocab_size"], [150, 97, 131], seed=8)
    refs = tt.plain_logits(w, cfg, seqs)
    names = list(seqs)
    first = {n: 3 + 5 * i for i, n in enumerate(names)}
    got = {n: [] for n in names}
    out = runner.step([StepEntry(n, seqs[n][:first[n]], range(first[n])) for n in names]).cpu().double()
    i = 0
    for n in names:
        got[n].append(out[i:i + first[n]])
        i += first[n]
    for t in range(1, 150):
        step = [n for n in names if first[n] + t - 1 < len(seqs[n])]
        if not step:
            break
        out = runner.step([StepEntry(n, [seqs[n][first[n] + t - 1]], [0]) for n in step]).cpu().double()
        for j, n in enumerate(step):
            got[n].append(out[j:j + 1])
    for n in names:
        rows = torch.cat(got[n])
        ref = refs[n][:rows.shape[0]]
        err = ((rows - ref).abs().amax(dim=1) / ref.abs().amax(dim=1)).max()
        assert float(err) <= 6e-2, f"{n}: worst relative error {float(err):.2e}"
        assert rows.shape[0] == len(seqs[n])


@pytest.mark.parametrize("name", ["tiny_d", "tiny_e"])
def test_steps_are_captured_per_count_of_slices_as_contexts_grow(tmp_path, cuda_device, monkeypatch, name):
    """The attention cuts the context of a decoded token into slices, how many it chooses from the
    batch and the longest live context, and it tags the step with the count: the runner keeps a
    captured step per (batch bucket, tags).  With the cost of a slice made small the count grows
    with the context within the 140 tokens decoded here (up to 16 slices over three tiles, most
    of them empty): every logit row of long decoding against the whole sequence, across the
    changes of kind."""
    import importlib
    R = importlib.import_module("gollmgo_b200.engine.runner")
    A = importlib.import_module("gollmgo_b200.parts.attention")
    monkeypatch.setattr(A, "PER_SLICE_US", 0.001)
    monkeypatch.setattr(A, "CLUSTER_OVERHEAD_US", 0.0)
    monkeypatch.setattr(A, "SPLIT_OVERHEAD_US", 0.01)
    A._decode_splits.cache_clear()
    from gollmgo_b200.config import EngineConfig
    from gollmgo_b200.engine.batch import StepEntry
    cfg, page, std, jitter = tiny_configs.get(name)
    d = tt.model_folder(str(tmp_path), name, cfg, seed=32, std=std, jitter=jitter, dtype="bfloat16")
    w = tt.load_weights(d)
    runner = R.load_runner(d, EngineConfig(dtype="bfloat16", block_size=page, num_blocks=96, max_batch_size=4,
                                           max_token_budget=64, max_model_len=256))
    mixer = runner.model.blocks[0].mixer
    assert mixer._splits(2, 40) < mixer._splits(2, 100) <= mixer._splits(2, 200)
    seqs = tt.random_requests(cfg["vocab_size"], [140, 90], seed=9)
    refs = tt.plain_logits(w, cfg, seqs)
    names = list(seqs)
    first = {n: 3 + 5 * i for i, n in enumerate(names)}
    got = {n: [] for n in names}
    out = runner.step([StepEntry(n, seqs[n][:first[n]], range(first[n])) for n in names]).cpu().double()
    i = 0
    for n in names:
        got[n].append(out[i:i + first[n]])
        i += first[n]
    for t in range(1, 140):
        step = [n for n in names if first[n] + t - 1 < len(seqs[n])]
        if not step:
            break
        out = runner.step([StepEntry(n, [seqs[n][first[n] + t - 1]], [0]) for n in step]).cpu().double()
        for j, n in enumerate(step):
            got[n].append(out[j:j + 1])
    kinds = [k for k in runner._graphs if isinstance(k, tuple)]
    assert len({tags for b, tags in kinds if b == 2}) >= 2, kinds            # batch 2 passed through several counts
    assert any(b == 1 for b, _ in kinds), kinds                               # and the last sequence alone too
    A._decode_splits.cache_clear()
    for n in names:
        rows = torch.cat(got[n])
        ref = refs[n][:rows.shape[0]]
        err = ((rows - ref).abs().amax(dim=1) / ref.abs().amax(dim=1)).max()
        assert float(err) <= 6e-2, f"{n}: worst relative error {float(err):.2e}"
        assert rows.shape[0] == len(seqs[n])


def test_decode_steps_of_every_batch_size_are_captured_when_the_engine_is_built(models):
    """No capture happens in the middle of generation, whatever batch sizes the requests pass
    through as they end one by one; an engine that captures at first use gives the same."""
    from gollmgo_b200 import Engine, SamplingParams
    from gollmgo_b200.engine.runner import GRAPH_BUCKETS
    d, cfg, page, w = models["tiny_a"]
    reqs = list(tt.random_requests(cfg["vocab_size"], [5, 9, 3, 11, 6], seed=9).values())
    eng = Engine(d, dtype="bfloat16", block_size=page, num_blocks=32, max_batch_size=6, max_token_budget=64)
    want = {b for b in GRAPH_BUCKETS if b <= 6}
    bucket_of = lambda key: key[0] if isinstance(key, tuple) else key
    assert {bucket_of(k) for k, c in eng.runner._graphs.items() if c.graph is not None} == want
    assert eng.runner.cache.free_pages() == 32 and not eng.runner.cache.requests
    graphs = {b: c.graph for b, c in eng.runner._graphs.items()}
    for i, r in enumerate(reqs):                               # different lengths: the batch shrinks step by step
        eng.enqueue(r, SamplingParams(max_tokens=4 + 3 * i, ignore_eos=True), request_id=f"r{i}")
    while eng.has_unfinished():
        eng.step()
    assert {b: c.graph for b, c in eng.runner._graphs.items()} == graphs
    lazy = Engine(d, dtype="bfloat16", block_size=page, num_blocks=32, max_batch_size=6, max_token_budget=64,
                  capture_at_start=False)
    assert not lazy.runner._graphs
    for i, r in enumerate(reqs):
        lazy.enqueue(r, SamplingParams(max_tokens=4 + 3 * i, ignore_eos=True), request_id=f"r{i}")
    while lazy.has_unfinished():
        lazy.step()
    for i in range(len(reqs)):
        assert lazy.output_of(f"r{i}").token_ids == eng.output_of(f"r{i}").token_ids


def test_small_pool_preempts_and_results_do_not_change(models):
    from gollmgo_b200 import Engine, SamplingParams
    d, cfg, page, w = models["tiny_a"]
    reqs = list(tt.random_requests(cfg["vocab_size"], [30, 12, 25, 7, 18], seed=4).values())
    params = SamplingParams(max_tokens=40, ignore_eos=True)
    roomy = Engine(d, dtype="float32", block_size=page, num_blocks=64, max_batch_size=8, max_token_budget=64)
    want = [o.token_ids for o in roomy.generate(reqs, params)]
    assert roomy.stats.preemptions == 0
    tight = Engine(d, dtype="float32", block_size=page, num_blocks=9, max_batch_size=8,
                   max_token_budget=40, prefill_chunk_size=16)
    outs = tight.generate(reqs, params)
    assert [o.token_ids for o in outs] == want
    assert tight.stats.preemptions > 0 and sum(o.preemptions for o in outs) == tight.stats.preemptions
    tight.runner.cache.audit()
    assert tight.runner.cache.free_pages() == 9
    assert want[0] == P.generate(w, cfg, reqs[0], 40, cast=torch.float32)


def test_requests_that_cannot_fit_are_refused(models):
    from gollmgo_b200 import Engine, SamplingParams
    from gollmgo_b200.engine import RequestTooLong
    d, cfg, page, w = models["tiny_a"]
    eng = Engine(d, dtype="float32", block_size=page, num_blocks=4, max_batch_size=2, max_token_budget=64)
    with pytest.raises(RequestTooLong):
        eng.enqueue(list(range(60)), SamplingParams(max_tokens=10))
    with pytest.raises(ValueError, match="outside"):
        eng.enqueue([1, 2, 9999], SamplingParams(max_tokens=2))


def test_command_line_generate_and_bench(models):
    d, cfg, page, w = models["tiny_a"]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    base = [sys.executable, "-m", "gollmgo_b200"]
    common = ["--model", d, "--dtype", "float32", "--block-size", str(page), "--num-blocks", "32",
              "--max-batch-size", "4", "--max-token-budget", "64", "--log-level", "error"]
    p = subprocess.run(base + ["generate", *common, "--prompt-ids", "5,6,7", "--prompt-ids", "9",
                               "--max-tokens", "5", "--ignore-eos"], capture_output=True, text=True, cwd=root)
    assert p.returncode == 0, p.stderr
    lines = [json.loads(l) for l in p.stdout.strip().splitlines()]
    assert lines[0]["token_ids"] == P.generate(w, cfg, [5, 6, 7], 5, cast=torch.float32)
    assert lines[1]["token_ids"] == P.generate(w, cfg, [9], 5, cast=torch.float32)
    p = subprocess.run(base + ["bench", *common, "--mode", "offline", "--num-prompts", "6", "--prompt-len", "10",
                               "--output-len", "4"], capture_output=True, text=True, cwd=root)
    assert p.returncode == 0, p.stderr
    res = json.loads(p.stdout)
    assert res["num_prompts"] == 6 and res["tokens_per_second"] > 0 and res["error_count"] == 0
    # lengths drawn from a seed: the same workload twice, every request served, the step counters kept
    runs = []
    for _ in range(2):
        p = subprocess.run(base + ["bench", *common, "--mode", "offline", "--num-prompts", "7", "--prompt-len-range",
                                   "3,20", "--output-len-range", "2,9", "--workload-seed", "5"],
                           capture_output=True, text=True, cwd=root)
        assert p.returncode == 0, p.stderr
        runs.append(json.loads(p.stdout))
    a, b = runs
    assert a["prompt_tokens"] == b["prompt_tokens"] and a["output_tokens"] == b["output_tokens"]
    assert 7 * 3 <= a["prompt_tokens"] <= 7 * 20 and 7 * 2 <= a["output_tokens"] <= 7 * 9
    assert a["engine_steps"] > 0 and 1 <= a["mean_batch"] <= 4 and a["pages_high_water"] > 0
    assert a["error_count"] == 0 and a["prompt_len_range"] == [3, 20]
    for mode, extra in (("decode", ["--batch", "3", "--context", "20", "--output-len", "8"]),
                        ("prefill", ["--prompt-len", "40"])):
        args = [a for a in common if a not in ("--num-blocks", "32")]
        p = subprocess.run(base + ["bench", *args, "--mode", mode, *extra], capture_output=True, text=True, cwd=root)
        assert p.returncode == 0, p.stderr
        res = json.loads(p.stdout)
        assert res["mode"] == mode and res["tokens_per_second"] > 0
