"""The plain implementation against TensorGreed/gollmgo's own engine.

tests/plain_llama.py restates the reference's formulas; here it is compared with what the
reference's unmodified CUDA code computes for a tiny random model (built and driven through
its C API by baseline/reference_arm.py, in a process of its own): one whole prompt through
gollmgo_model_forward (kernels/gollmgo_model.cu:862-899), and prefill + single-sequence decode
through gollmgo_model_forward_prefill / _forward_paged (:901-1063).  The reference rounds every
activation and its logits to bfloat16, so the comparison is at the bfloat16 tolerance of the
other tests.  The configuration is one that the reference computes as config.json says (see
tests/golden/make_reference_anchor.py).

Without a GPU the same comparison runs against the committed output of that script, if there."""
import os
import sys

import numpy as np
import pytest
import torch

import plain_llama

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import make_reference_anchor as anchor  # noqa: E402

TOL = 4e-2


def plain_side():
    w, tokens = anchor.inputs()
    weights = {k: torch.from_numpy(anchor.bits_to_float(v).copy()).reshape(v.shape) for k, v in w.items()}
    return plain_llama.forward(weights, anchor.CONFIG, tokens.tolist()).numpy(), tokens


def check(ref):
    plain, tokens = plain_side()
    assert ref["whole"].shape == plain.shape

    def worst(got, want):
        assert np.isfinite(got).all()
        return float((np.abs(got - want).max(axis=1) / np.abs(want).max(axis=1)).max())
    e_whole = worst(ref["whole"], plain)
    e_prefill = worst(ref["prefill"], plain[:anchor.N_PREFILL])
    e_paged = worst(ref["paged"], plain[anchor.N_PREFILL - 1:])
    assert max(e_whole, e_prefill, e_paged) <= TOL, (e_whole, e_prefill, e_paged)
    # and it chooses the same next token wherever the plain logits have a clear winner
    agree = total = 0
    for got, want in zip(ref["whole"], plain):
        top = np.sort(want)[-2:]
        if top[1] - top[0] > 2.5 * TOL * np.abs(want).max():
            total += 1
            agree += int(got.argmax() == want.argmax())
    assert total >= 5 and agree == total
    return e_whole, e_prefill, e_paged


@pytest.mark.gpu
def test_plain_implementation_matches_the_reference_engine(tmp_path, cuda_device):
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline"))
    import reference_arm as ra
    try:
        ra.build()
    except ra.Unavailable as exc:
        pytest.skip(f"the reference cannot be built here: {exc}")
    ref = anchor.run_reference(str(tmp_path / "out.npz"), str(tmp_path))
    errs = check(ref)
    print("plain vs reference (whole, prefill, paged decode): " + ", ".join(f"{e:.2e}" for e in errs))


def test_plain_implementation_matches_the_committed_reference_output():
    if not os.path.exists(anchor.GOLDEN):
        pytest.skip("no committed reference output")
    check(np.load(anchor.GOLDEN))
