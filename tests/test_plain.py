"""The plain implementation checked against facts that do not depend on it:
hand-computed values, invariances, and the host-side formulas of the package."""
import math

import pytest
import torch

import plain_llama as P
import tiny_configs
from gollmgo_b200.config import RopeScaling
from gollmgo_b200.parts.position import inverse_frequencies


def test_rms_norm_by_hand():
    x = torch.tensor([[3.0, 4.0]])
    y = P.rms_norm(x, torch.tensor([2.0, 0.5]), 0.0)
    r = 1.0 / math.sqrt((9 + 16) / 2)
    assert torch.allclose(y, torch.tensor([[3 * r * 2, 4 * r * 0.5]], dtype=torch.float64))


def test_rope_half_split_and_adjacent_by_hand():
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0]]])            # one token, one head, d = 4
    f = torch.tensor([1.0, 0.5], dtype=torch.float64)
    pos = torch.tensor([2])
    h = P.apply_rope(x, pos, f)[0, 0]                      # pairs (0,2) and (1,3)
    c0, s0, c1, s1 = math.cos(2.0), math.sin(2.0), math.cos(1.0), math.sin(1.0)
    assert torch.allclose(h, torch.tensor([1 * c0 - 3 * s0, 2 * c1 - 4 * s1, 1 * s0 + 3 * c0, 2 * s1 + 4 * c1], dtype=torch.float64))
    a = P.apply_rope(x, pos, f, interleaved=True)[0, 0]    # pairs (0,1) and (2,3)
    assert torch.allclose(a, torch.tensor([1 * c0 - 2 * s0, 1 * s0 + 2 * c0, 3 * c1 - 4 * s1, 3 * s1 + 4 * c1], dtype=torch.float64))
    assert torch.allclose(P.apply_rope(x, torch.tensor([0]), f), x.double())


def test_llama3_scaling_regions():
    sc = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 64}
    base = P.rope_inv_freq(32, 500000.0, None)
    f = P.rope_inv_freq(32, 500000.0, sc)
    wl = 2 * math.pi / base
    assert torch.equal(f[wl < 16], base[wl < 16])                      # short waves kept
    assert torch.allclose(f[wl > 64], base[wl > 64] / 8)               # long waves slowed
    mid = (wl >= 16) & (wl <= 64)
    assert mid.any() and ((f[mid] < base[mid]) & (f[mid] > base[mid] / 8)).all()
    # the package's own table builder agrees (written separately)
    ours = inverse_frequencies(32, 500000.0, RopeScaling("llama3", 8.0, 1.0, 4.0, 64))
    assert torch.allclose(ours, f, rtol=1e-14, atol=0)
    assert torch.allclose(inverse_frequencies(16, 10000.0, None), P.rope_inv_freq(16, 10000.0, None), rtol=1e-14, atol=0)


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    T, nh, nkv, d = 9, 4, 2, 8
    q, k, v = torch.randn(T, nh, d), torch.randn(T, nkv, d), torch.randn(T, nkv, d)
    o = P.attention(q, k, v)
    o2 = P.attention(q[:5], k[:5], v[:5])
    assert torch.allclose(o[:5], o2)                                   # later tokens change nothing earlier
    assert torch.allclose(o[0, 1], v[0, 0].double())                   # first token sees only itself; head 1 -> kv 0
    assert torch.allclose(o[0, 2], v[0, 1].double())                   # head 2 -> kv head 1
    w1 = P.attention(q, k, v, window=1)
    assert torch.allclose(w1[:, 3], v[:, 1].double())                  # window 1: only itself
    k2 = k.clone()
    k2[0] += 100.0                                                     # token 0 is outside a window of 3 for i >= 3
    assert torch.allclose(P.attention(q, k2, v, window=3)[3:], P.attention(q, k, v, window=3)[3:])


def test_forward_prefix_consistency_and_tied_head():
    from gollmgo_b200.parts import manifest_for_config
    from gollmgo_b200.weights import random_tensor
    for name in ("tiny_a", "tiny_b", "tiny_c"):
        cfg, _, std, jitter = tiny_configs.get(name)
        w = {n: random_tensor(n, s, 1, "cpu", torch.float32, std, jitter)
             for n, s in manifest_for_config(cfg).items() if not s.optional}
        toks = list(range(3, 40))
        full = P.forward(w, cfg, toks)
        assert full.shape == (37, cfg["vocab_size"]) and torch.isfinite(full).all()
        assert torch.allclose(full[:11], P.forward(w, cfg, toks[:11]), atol=1e-10)
        assert float(full.std()) > 0.05                                # the weights give logits that tell tokens apart


def test_sampling_by_hand():
    assert P.argmax([1.0, 3.0, 3.0, 2.0]) == 1                         # first maximum wins
    p = P.probabilities([0.0, math.log(2.0), math.log(4.0), -50.0], 1.0)
    assert torch.allclose(p[:3], torch.tensor([1 / 7, 2 / 7, 4 / 7], dtype=torch.float64), atol=1e-9)
    pk = P.probabilities([0.0, math.log(2.0), math.log(4.0), -50.0], 1.0, top_k=2)
    assert torch.allclose(pk, torch.tensor([0, 1 / 3, 2 / 3, 0], dtype=torch.float64), atol=1e-9)
    pp = P.probabilities([0.0, math.log(2.0), math.log(4.0), -50.0], 1.0, top_p=0.6)
    assert torch.allclose(pp, torch.tensor([0, 1 / 3, 2 / 3, 0], dtype=torch.float64), atol=1e-9)   # 4/7 < .6 <= 6/7
    pt = P.probabilities([0.0, 2.0], 2.0)
    assert torch.allclose(pt[1] / pt[0], torch.tensor(math.e, dtype=torch.float64))
    assert P.categorical(torch.tensor([0.25, 0.25, 0.5]), 0.49) == 1
    assert P.categorical(torch.tensor([0.25, 0.25, 0.5]), 0.5) == 2
    assert P.categorical(torch.tensor([0.5, 0.5, 0.0]), 0.999999999999) == 1
    us = [P.uniform_draw(7, n) for n in range(2000)]
    assert all(0 <= u < 1 for u in us) and abs(sum(us) / len(us) - 0.5) < 0.03
    assert P.uniform_draw(7, 3) == P.uniform_draw(7, 3) != P.uniform_draw(8, 3)
    assert P.sample([0.1, 0.9, 0.3], 0.0, seed=1, n=0) == 1
