"""The layer sizes of the headline configuration (hidden 4096, 32/8 heads of 128, feed-forward
14336, vocabulary 128256; two layers, random weights): the same 1500 tokens as one step and cut
into portions down to one token must give the same logits, in float32 and in bfloat16.  The tiny
configurations cannot reach the paths that only these sizes take (several waves of tiles in the
tcgen05 kernels, the weight-streaming products over long rows, 16 KB rows in the norm)."""
import json
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPE = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                     "gollmgo_b200", "bench_shapes", "llama_3_1_8b.json")


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 4e-2)])
def test_whole_prompt_equals_portions_at_full_width(cuda_device, dtype, tol):
    from gollmgo_b200.config import EngineConfig
    from gollmgo_b200.engine.batch import StepEntry
    from gollmgo_b200.engine.runner import ModelRunner
    with open(SHAPE) as f:
        cfg = json.load(f)
    cfg["num_hidden_layers"] = 2
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(0, cfg["vocab_size"], (1500,), generator=g).tolist()
    runner = ModelRunner(cfg, EngineConfig(dtype=dtype, block_size=16, num_blocks=512, max_batch_size=8,
                                           max_token_budget=2048, max_model_len=4096), weights_seed=1)
    want = list(range(0, 1500, 97)) + [1499]
    whole = runner.step([StepEntry("w", toks, want)]).float().cpu()
    runner.check_kernels()
    rows, pos = [], 0
    for n in (1100, 128, 100, 2, 70, 1, 1, 98):
        w = [p - pos for p in want if pos <= p < pos + n]
        out = runner.step([StepEntry("c", toks[pos:pos + n], w)])
        if w:
            rows.append(out.float().cpu())
        pos += n
    runner.check_kernels()
    cut = torch.cat(rows)
    assert torch.isfinite(whole).all() and float(whole.abs().max()) > 1.0
    err = float(((whole - cut).abs().amax(1) / whole.abs().amax(1)).max())
    assert err <= tol, f"worst relative error {err:.2e}"
    runner.release("w"), runner.release("c")
    runner.cache.audit()
