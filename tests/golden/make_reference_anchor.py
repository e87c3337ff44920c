"""Makes tests/golden/reference_anchor.npz: what TensorGreed/gollmgo's own CUDA engine computes
for a tiny random Llama model, so that the plain implementation (tests/plain_llama.py) can be
compared with the reference's output where no GPU is at hand.

    python tests/golden/make_reference_anchor.py            (on a machine with a CUDA device)

The reference cannot run on a CPU (CUDA + cuBLAS), so this is run on the GPU box once and its
small output is committed.  It builds the reference's kernels/*.cu unmodified and calls its C
API (baseline/reference_arm.py::run_anchor): one whole prompt through gollmgo_model_forward,
and the same tokens through gollmgo_model_forward_prefill followed by single-sequence decode
steps through gollmgo_model_forward_paged.

The configuration is one the reference computes as config.json says: rotary pairs adjacent
(``rope_interleaved``), theta 10000 (it hard-codes both: kernels/gollmgo_ops.cu:321-358,
kernels/gollmgo_model.cu:603-606), untied head, eps as passed; head size 32 so that its
one-warp attention blocks are full warps.
"""
import json
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
GOLDEN = os.path.join(HERE, "reference_anchor.npz")

CONFIG = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 128, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 32, "intermediate_size": 192, "vocab_size": 256,
    "rope_theta": 10000.0, "rope_interleaved": True, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "max_position_embeddings": 512, "hidden_act": "silu",
}
N_TOKENS, N_PREFILL = 44, 33


def bf16_bits(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bits_to_float(b):
    return (b.astype(np.uint32) << 16).view(np.float32)


def inputs(seed=17):
    """Weights (bfloat16 bit patterns by tensor name) and tokens, from a seed."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm as ra
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in ra.tensor_names(CONFIG):
        if len(shape) == 1:
            w[name] = bf16_bits(1.0 + 0.1 * rng.standard_normal(shape))
        else:
            w[name] = bf16_bits(0.09 * rng.standard_normal(shape)).reshape(shape)
    tokens = rng.integers(0, CONFIG["vocab_size"], N_TOKENS).astype(np.int32)
    return w, tokens


def run_reference(out_npz, workdir):
    w, tokens = inputs()
    in_npz = os.path.join(workdir, "anchor_in.npz")
    np.savez(in_npz, config=json.dumps(CONFIG), tokens=tokens, n_prefill=N_PREFILL, **w)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "baseline", "reference_arm.py"), "anchor", in_npz, out_npz],
                       capture_output=True, text=True, timeout=600)
    if p.returncode != 0:
        raise RuntimeError(f"the reference did not run: {(p.stderr or p.stdout)[-600:]}")
    return np.load(out_npz)


if __name__ == "__main__":
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        out = run_reference(os.path.join(tmp, "o.npz"), tmp)
        np.savez_compressed(GOLDEN, whole=out["whole"], paged=out["paged"], prefill=out["prefill"])
    print(f"wrote {GOLDEN}")
