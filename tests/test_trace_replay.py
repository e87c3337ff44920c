"""Replay through bin/trace_run, compared with the plain implementation: the same
requests whole, with the last 32 tokens one by one, in portions of changing size,
and mixed with other requests on a pool so small that pages are used again; in
float32 and in bfloat16; for tiny configurations that differ in every size."""
import pytest
import torch

import tiny_configs
import trace_tools as tt

pytestmark = pytest.mark.gpu

LENGTHS = {"tiny_a": [7, 13, 1, 70, 45, 101], "tiny_b": [1, 5, 37, 70, 130, 96],
           "tiny_c": [3, 66, 40, 150, 97, 129], "tiny_d": [2, 64, 65, 130, 200, 33],
           "tiny_e": [1, 129, 64, 190, 80, 257]}
TOL = {"float32": 2e-5, "bfloat16": 4e-2}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c", "tiny_d", "tiny_e"])
def test_replay_matches_plain(tmp_path, cuda_device, name, dtype):
    config, page, std, jitter = tiny_configs.get(name)
    model_dir = tt.model_folder(str(tmp_path), name, config, seed=11, std=std, jitter=jitter,
                                dtype="float32" if dtype == "float32" else "bfloat16")
    weights = tt.load_weights(model_dir)
    requests = tt.random_requests(config["vocab_size"], LENGTHS[name], seed=5)
    reference = tt.plain_logits(weights, config, requests)
    trace = tt.Trace()
    tt.whole(trace, requests)
    tt.tail_decode(trace, requests)
    tt.portions(trace, requests)
    peak_single = trace.peak
    tt.mixed(trace, requests, max_live=4, seed=3)
    tt.mixed(trace, dict(reversed(list(requests.items()))), max_live=3, seed=4, tag="n")
    out = str(tmp_path / "out")
    tt.run_trace(model_dir, dtype, trace, out, block_size=page)
    worst = tt.compare(trace, out, reference, config["vocab_size"], TOL[dtype])
    pool, asked, shared = tt.pages_were_used_again(trace, out + "/pages.jsonl", page)
    print(f"{name} {dtype}: {len(trace.steps)} steps, pool {trace.peak} tokens = {pool} pages for {asked} "
          f"pages asked in all, {shared} page ids held by several requests "
          f"(single-request peak {peak_single}), worst relative error {worst:.2e}")


@pytest.mark.parametrize("name,dtype", [("tiny_b", "bfloat16"), ("tiny_c", "bfloat16"), ("tiny_e", "bfloat16"),
                                        ("tiny_c", "float32")])
def test_pages_given_back_are_never_read(tmp_path, cuda_device, name, dtype):
    """The mixed trace on a small pool with every page overwritten by NaN the moment it is given
    back (finished requests, pages behind a window): a kernel that read a page its request no
    longer holds, or beyond a request's context inside a page, would produce NaN logits."""
    import os
    config, page, std, jitter = tiny_configs.get(name)
    model_dir = tt.model_folder(str(tmp_path), name, config, seed=12, std=std, jitter=jitter,
                                dtype="float32" if dtype == "float32" else "bfloat16")
    weights = tt.load_weights(model_dir)
    requests = tt.random_requests(config["vocab_size"], LENGTHS[name], seed=6)
    reference = tt.plain_logits(weights, config, requests)
    trace = tt.Trace()
    tt.mixed(trace, requests, max_live=4, seed=7)
    tt.portions(trace, requests)
    tt.mixed(trace, dict(reversed(list(requests.items()))), max_live=3, seed=8, tag="n")
    out = str(tmp_path / "out")
    env = dict(os.environ, GOLLMGO_B200_POISON_FREED="1")
    tt.run_trace(model_dir, dtype, trace, out, block_size=page, env=env)
    tt.compare(trace, out, reference, config["vocab_size"], TOL[dtype])
    tt.pages_were_used_again(trace, out + "/pages.jsonl", page)
