"""Plain, slow implementation of the Llama dense decoder. The oracle of the tests.

Whole sequences, no cache, no paging, no batching: one function for each part,
written from the formulas of TensorGreed/gollmgo's CUDA model (cited per
function as file:line within that project). It shares no code with the
``gollmgo_b200`` package: it takes a plain dict of tensors keyed by their
safetensors names and the raw ``config.json`` dict.

gollmgo's own model code cannot be built on a CPU (it is CUDA + cuBLAS behind a
Go host program, and the only CPU code it has are three formula helpers in
``kernels/gollmgo_ops_test.cu:38-87``), so this file is written from the formulas.
It is then compared with a run of the reference's unmodified CUDA engine on a
GPU: ``tests/golden/make_reference_anchor.py`` made ``tests/golden/reference_anchor.npz``
(a tiny random model through gollmgo_model_forward, and through prefill + paged
decode), and ``tests/test_reference_anchor.py`` checks this file against it, with
or without a GPU.

Where the reference ignores a config.json key (rope_theta, rms_norm_eps,
rope_scaling, tie_word_embeddings, head_dim) the key is honoured here, because
the engine reads every size and constant from config.json.  The rotary pairing
is the half-split layout ``(p, p + d/2)`` that tensors with these names are
stored for; ``rope_interleaved: true`` selects the reference's adjacent pairs
``(2p, 2p+1)`` (kernels/gollmgo_ops.cu:321-358).

All arithmetic is float64 unless ``dtype`` says otherwise, so that it is the
most exact thing in the comparison.  ``forward(..., device=...)`` does the same
arithmetic on that device (the weights stay where they are and are brought over
tensor by tensor), which is what makes the layer sizes of a real checkpoint
affordable; ``rows`` limits the head product to the positions that are compared.
"""
from __future__ import annotations

import math

import torch


# --------------------------------------------------------------------------- parts

def embed(table: torch.Tensor, ids) -> torch.Tensor:
    """x0[t, :] = float(E[id_t, :])  -- kernels/gollmgo_ops.cu:538-552."""
    ids = torch.as_tensor(ids, dtype=torch.long, device=table.device)
    return table[ids].to(torch.float64)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w  -- kernels/gollmgo_ops.cu:593-629."""
    x = x.to(torch.float64)
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(ms + eps) * weight.to(torch.float64)


def rope_inv_freq(head_dim: int, theta: float, scaling: dict | None) -> torch.Tensor:
    """f_p = 1 / theta^(2p/d) for p in [0, d/2)  -- kernels/gollmgo_ops.cu:337.

    With ``rope_scaling`` of type llama3 (a key the reference does not read)
    long wavelengths are stretched: wavelength 2*pi/f below orig/high keeps f,
    above orig/low uses f/factor, between the two blends linearly.
    """
    half = head_dim // 2
    f = [1.0 / (theta ** (2.0 * p / head_dim)) for p in range(half)]
    if scaling:
        kind = scaling.get("rope_type", scaling.get("type"))
        if kind == "llama3":
            factor = float(scaling["factor"])
            low = float(scaling["low_freq_factor"])
            high = float(scaling["high_freq_factor"])
            orig = float(scaling["original_max_position_embeddings"])
            out = []
            for fp in f:
                wavelen = 2.0 * math.pi / fp
                if wavelen < orig / high:
                    out.append(fp)
                elif wavelen > orig / low:
                    out.append(fp / factor)
                else:
                    s = (orig / wavelen - low) / (high - low)
                    out.append((1.0 - s) * fp / factor + s * fp)
            f = out
        elif kind == "linear":
            f = [fp / float(scaling["factor"]) for fp in f]
        elif kind not in (None, "default"):
            raise ValueError(f"plain implementation: rope_scaling type {kind!r}")
    return torch.tensor(f, dtype=torch.float64)


def apply_rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor,
               interleaved: bool = False) -> torch.Tensor:
    """Rotate pairs of x[t, h, :] by angle pos*f_p  -- kernels/gollmgo_ops.cu:336-357.

    (a, b) <- (a cos - b sin, a sin + b cos); pairs are (p, p+d/2), or
    (2p, 2p+1) when ``interleaved``.
    """
    x = x.to(torch.float64)
    d = x.shape[-1]
    half = d // 2
    ang = positions.to(x.device, torch.float64)[:, None] * inv_freq.to(x.device)[None, :]   # [T, d/2]
    cos = torch.cos(ang)[:, None, :]
    sin = torch.sin(ang)[:, None, :]
    out = torch.empty_like(x)
    if interleaved:
        a, b = x[..., 0::2], x[..., 1::2]
        out[..., 0::2] = a * cos - b * sin
        out[..., 1::2] = a * sin + b * cos
    else:
        a, b = x[..., :half], x[..., half:]
        out[..., :half] = a * cos - b * sin
        out[..., half:] = a * sin + b * cos
    return out


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
              window: int | None = None) -> torch.Tensor:
    """Causal grouped-query attention of one whole sequence.

    kv head of q head h is h // (nh/nkv); s_ij = (q_i . k_j) / sqrt(d) for
    j <= i; softmax over j; o_i = sum_j p_ij v_j
    -- kernels/gollmgo_ops.cu:377-446 and kernels/gollmgo_paged_attn.cu:149-223.
    ``window`` (not in the reference) keeps only j > i - window.
    q: [T, nh, d], k, v: [T, nkv, d] -> [T, nh, d]
    """
    T, nh, d = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    scale = 1.0 / math.sqrt(d)
    out = torch.zeros(T, nh, d, dtype=torch.float64, device=q.device)
    i_idx = torch.arange(T, device=q.device)[:, None]
    j_idx = torch.arange(T, device=q.device)[None, :]
    allowed = j_idx <= i_idx
    if window is not None:
        allowed &= j_idx > i_idx - window
    for h in range(nh):
        kh = h // group
        s = (q[:, h, :].to(torch.float64) @ k[:, kh, :].to(torch.float64).T) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        e = torch.exp(s - m)
        p = e / e.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ v[:, kh, :].to(torch.float64)
    return out


def gated_mlp(x: torch.Tensor, w_gate, w_up, w_down) -> torch.Tensor:
    """down( silu(x Wg^T) * (x Wu^T) ), silu(g) = g / (1 + exp(-g))
    -- kernels/gollmgo_model.cu:746-776, kernels/gollmgo_ops.cu:361-374."""
    x = x.to(torch.float64)
    g = x @ w_gate.to(torch.float64).T
    u = x @ w_up.to(torch.float64).T
    a = g / (1.0 + torch.exp(-g)) * u
    return a @ w_down.to(torch.float64).T


# --------------------------------------------------------------------------- model

def _cfg(config: dict):
    nh = config["num_attention_heads"]
    nkv = config.get("num_key_value_heads") or nh
    d = config.get("head_dim") or config["hidden_size"] // nh
    return nh, nkv, d


def layer_windows(config: dict) -> list:
    """Per-layer attention window (None = all keys).  Keys ``sliding_window`` and
    ``layer_types`` are optional; plain Llama has neither."""
    L = config["num_hidden_layers"]
    win = config.get("sliding_window")
    types = config.get("layer_types")
    if not win:
        return [None] * L
    if types is None:
        return [win] * L
    return [win if t == "sliding_attention" else None for t in types]


class _On:
    """The weights dict, each tensor brought to ``device`` when it is asked for."""

    def __init__(self, w, device):
        self.w, self.device = w, device

    def __getitem__(self, name):
        return self.w[name].to(self.device)


def decoder_layer(x, w: dict, l: int, config: dict, positions, inv_freq, window):
    """One pre-norm block: x += Wo attn(rope(q), rope(k), v); x += mlp(norm(x))
    -- kernels/gollmgo_model.cu:551-792 (run_layer)."""
    nh, nkv, d = _cfg(config)
    eps = config.get("rms_norm_eps", 1e-5)
    p = f"model.layers.{l}."
    T = x.shape[0]
    w = _On(w, x.device)
    h = rms_norm(x, w[p + "input_layernorm.weight"], eps)
    q = (h @ w[p + "self_attn.q_proj.weight"].to(torch.float64).T).view(T, nh, d)
    k = (h @ w[p + "self_attn.k_proj.weight"].to(torch.float64).T).view(T, nkv, d)
    v = (h @ w[p + "self_attn.v_proj.weight"].to(torch.float64).T).view(T, nkv, d)
    inter = bool(config.get("rope_interleaved", False))
    q = apply_rope(q, positions, inv_freq, inter)
    k = apply_rope(k, positions, inv_freq, inter)
    a = attention(q, k, v, window).reshape(T, nh * d)
    x = x + a @ w[p + "self_attn.o_proj.weight"].to(torch.float64).T
    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
    x = x + gated_mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                      w[p + "mlp.down_proj.weight"])
    return x


def forward(w: dict, config: dict, token_ids, device=None, rows=None) -> torch.Tensor:
    """Logits [T, V] (float64) of one whole sequence starting at position 0
    -- kernels/gollmgo_model.cu:862-899 (gollmgo_model_forward).  With ``rows`` only the
    logits at those positions, [len(rows), V]; with ``device`` the arithmetic runs there."""
    nh, nkv, d = _cfg(config)
    T = len(token_ids)
    dev = torch.device(device) if device is not None else w["model.embed_tokens.weight"].device
    positions = torch.arange(T, device=dev)
    inv_freq = rope_inv_freq(d, float(config.get("rope_theta", 10000.0)),
                             config.get("rope_scaling")).to(dev)
    windows = layer_windows(config)
    x = embed(w["model.embed_tokens.weight"], token_ids).to(dev)
    for l in range(config["num_hidden_layers"]):
        x = decoder_layer(x, w, l, config, positions, inv_freq, windows[l])
    if rows is not None:
        x = x[torch.as_tensor(list(rows), dtype=torch.long, device=dev)]
    x = rms_norm(x, w["model.norm.weight"].to(dev), config.get("rms_norm_eps", 1e-5))
    head = w["model.embed_tokens.weight"] if config.get("tie_word_embeddings", False) \
        else w["lm_head.weight"]
    return x @ head.to(dev).to(torch.float64).T


# --------------------------------------------------------------------------- sampling

def argmax(logits) -> int:
    """First maximum wins -- internal/engine/sampling.go:75-85."""
    best, best_val = 0, float(logits[0])
    for i in range(1, len(logits)):
        if float(logits[i]) > best_val:
            best, best_val = i, float(logits[i])
    return best


def uniform_draw(seed: int, n: int) -> float:
    """Draw number ``n`` of the request whose seed is ``seed``: a counter-based
    generator (splitmix64 of seed + (n+1)*golden), top 24 bits -> [0, 1).  The
    reference draws from one PCG stream per engine (internal/engine/sampling.go:29-37),
    which makes a request's tokens depend on its neighbours; this one does not."""
    mask = (1 << 64) - 1
    z = (seed + (n + 1) * 0x9E3779B97F4A7C15) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    z = z ^ (z >> 31)
    return (z >> 40) / float(1 << 24)


def probabilities(logits, temperature: float, top_k: int = 0, top_p: float = 0.0):
    """softmax(logits / T) after top-k, then top-p with renormalisation
    -- internal/engine/sampling.go:40-72, 88-173."""
    x = torch.as_tensor(logits, dtype=torch.float64) / temperature
    V = x.numel()
    if 0 < top_k < V:
        order = torch.sort(x, descending=True, stable=True).indices
        keep = torch.zeros(V, dtype=torch.bool)
        keep[order[:top_k]] = True
        x = x.masked_fill(~keep, float("-inf"))
    e = torch.exp(x - x.max())
    p = e / e.sum()
    if 0.0 < top_p < 1.0:
        order = torch.sort(p, descending=True, stable=True).indices
        kept = torch.zeros(V, dtype=torch.float64)
        cum = 0.0
        for i in order.tolist():
            if cum >= top_p and cum > 0:
                break
            kept[i] = p[i]
            cum += float(p[i])
        p = kept / kept.sum()
    return p


def categorical(p, u: float) -> int:
    """First index whose running sum exceeds u; fallback last non-zero
    -- internal/engine/sampling.go:176-192."""
    cum = 0.0
    for i, pi in enumerate(p.tolist()):
        cum += pi
        if u < cum:
            return i
    nz = torch.nonzero(p).flatten()
    return int(nz[-1]) if len(nz) else 0


def sample(logits, temperature: float, seed: int, n: int, top_k: int = 0, top_p: float = 0.0) -> int:
    if temperature <= 1e-9:
        return argmax(logits)
    return categorical(probabilities(logits, temperature, top_k, top_p), uniform_draw(seed, n))


def generate(w: dict, config: dict, prompt, max_new_tokens: int, temperature: float = 0.0,
             seed: int = 0, top_k: int = 0, top_p: float = 0.0, eos=None, cast=None):
    """Generate by running the whole sequence again for every token.  ``cast``
    rounds the logits the way the engine delivers them (e.g. to float32)."""
    toks = list(prompt)
    out = []
    for n in range(max_new_tokens):
        logits = forward(w, config, toks)[-1]
        if cast is not None:
            logits = logits.to(cast)
        t = sample(logits, temperature, seed, n, top_k, top_p)
        out.append(t)
        toks.append(t)
        if eos is not None and t in eos:
            break
    return out
