"""Toy parts defined HERE and registered from outside the package: a feed-forward with
routing (two experts, top-1 router in float32), another position encoding (a learned
per-position scale of q and k), and another block arrangement (mixer and feed-forward in
parallel on one norm).  A toy architecture uses them in different layers of one model; it is
built from a config, given random weights, stepped whole and in portions, and compared with a
plain computation.  None of this is a model of anyone's; it shows that the parts are general."""
import os

import pytest
import torch
from safetensors.torch import load_file

import plain_llama as P

pytestmark = pytest.mark.gpu

H, NH, NKV, D, I, V, E, MAXPOS = 48, 3, 3, 16, 64, 83, 2, 128


class RoutedFeedForward:
    """Top-1 of E gated experts per token; router logits and choice in float32."""

    def __init__(self, spec, ctx):
        self.hidden, self.inter, self.experts = int(spec["hidden_size"]), int(spec["intermediate_size"]), int(spec["experts"])
        self.ctx = ctx

    def weights(self):
        from gollmgo_b200.weights import WeightSpec
        w = {"router.weight": WeightSpec((self.experts, self.hidden))}
        for e in range(self.experts):
            w[f"experts.{e}.gate_proj.weight"] = WeightSpec((self.inter, self.hidden))
            w[f"experts.{e}.up_proj.weight"] = WeightSpec((self.inter, self.hidden))
            w[f"experts.{e}.down_proj.weight"] = WeightSpec((self.hidden, self.inter))
        return w

    def load(self, get):
        self.w = {n: get(n).float() for n in self.weights()}

    def forward(self, x, batch):
        xf = x.float()
        choice = (xf @ self.w["router.weight"].T).argmax(dim=-1)
        out = torch.zeros_like(xf)
        for e in range(self.experts):
            rows = (choice == e).nonzero().flatten()
            if rows.numel():
                h = xf[rows]
                g = h @ self.w[f"experts.{e}.gate_proj.weight"].T
                u = h @ self.w[f"experts.{e}.up_proj.weight"].T
                out[rows] = (g / (1 + torch.exp(-g)) * u) @ self.w[f"experts.{e}.down_proj.weight"].T
        return out.to(x.dtype)


class LearnedScalePositions:
    """q and k of the token at position p are multiplied by 1 + 0.5 * sin(p * freq_c) per channel c."""
    interleaved = False

    def __init__(self, spec, ctx):
        self.freq = torch.linspace(0.05, 0.4, int(spec["head_dim"]), device=ctx.device)

    def rope_table(self):
        return None

    def apply(self, qkv, batch, nh, nkv, d):
        T = qkv.shape[0]
        scale = 1 + 0.5 * torch.sin(batch.positions[:T].float()[:, None] * self.freq[None, :])      # [T, d]
        qk = qkv.view(T, nh + 2 * nkv, d)[:, :nh + nkv]
        qk.copy_((qk.float() * scale[:, None, :]).to(qkv.dtype))


class ParallelBlock:
    """x += mixer(norm(x)) + ffn(norm(x)): both read the same normed input."""

    def __init__(self, layer_spec, mixer, feed_forward, mixer_norm, ffn_norm, ctx):
        self.mixer, self.ff, self.norm, self.ctx, self.hidden = mixer, feed_forward, mixer_norm, ctx, mixer_norm.size
        ctx.workspace.reserve("toy_normed", ctx.max_tokens * self.hidden, ctx.act_dtype)

    def forward(self, resid, delta, batch, cache, writes_cache=True):
        T = resid.shape[0]
        h = self.ctx.workspace.get("toy_normed", T, self.hidden)
        self.norm.add_norm(resid, delta, h)
        a = self.mixer.forward(h, batch, cache, writes_cache)
        f = self.ff.forward(h, batch)
        return (a.float() + f.float()).to(a.dtype)


def toy_spec(cfg):
    from gollmgo_b200.parts import LayerSpec, ModelSpec, PartSpec, RunEntry
    norm = PartSpec("rmsnorm", {"size": H, "eps": 1e-5})
    rope = PartSpec("rope", {"head_dim": D, "theta": 10000.0, "scaling": None})
    learned = PartSpec("toy_learned_scale", {"head_dim": D})

    def attn(pos):
        return PartSpec("attention", {"hidden_size": H, "num_heads": NH, "num_kv_heads": NKV, "head_dim": D,
                                      "window": None, "position": pos})
    dense = PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": I})
    routed = PartSpec("toy_routed", {"hidden_size": H, "intermediate_size": I, "experts": E})

    def layer(i, block, mixer, ff):
        return LayerSpec(PartSpec(block), mixer, ff, norm, norm, mixer_prefix=f"t.{i}.mix.", ffn_prefix=f"t.{i}.ff.",
                         mixer_norm_name=f"t.{i}.n1", ffn_norm_name=f"t.{i}.n2")
    layers = (layer(0, "pre_norm", attn(learned), routed), layer(1, "toy_parallel", attn(rope), dense))
    return ModelSpec("ToyPartsForCausalLM", V, H, layers, (RunEntry(0, 0), RunEntry(1, 1)), norm, True,
                     "t.embed", "t.norm", "t.head", MAXPOS)


def plain(w, toks):
    T = len(toks)
    pos = torch.arange(T)
    x = P.embed(w["t.embed"], toks)

    def qkv(i, h):
        return ((h @ w[f"t.{i}.mix.q_proj.weight"].double().T).view(T, NH, D),
                (h @ w[f"t.{i}.mix.k_proj.weight"].double().T).view(T, NKV, D),
                (h @ w[f"t.{i}.mix.v_proj.weight"].double().T).view(T, NKV, D))
    # layer 0: learned-scale positions, routed feed-forward, pre-norm
    h = P.rms_norm(x, w["t.0.n1"], 1e-5)
    q, k, v = qkv(0, h)
    scale = (1 + 0.5 * torch.sin(pos.double()[:, None] * torch.linspace(0.05, 0.4, D).double()[None, :]))[:, None, :]
    x = x + P.attention(q * scale, k * scale, v).reshape(T, NH * D) @ w["t.0.mix.o_proj.weight"].double().T
    h = P.rms_norm(x, w["t.0.n2"], 1e-5)
    choice = (h @ w["t.0.ff.router.weight"].double().T).argmax(dim=-1)
    y = torch.zeros_like(h)
    for e in range(E):
        rows = (choice == e).nonzero().flatten()
        if rows.numel():
            y[rows] = P.gated_mlp(h[rows], w[f"t.0.ff.experts.{e}.gate_proj.weight"], w[f"t.0.ff.experts.{e}.up_proj.weight"],
                                  w[f"t.0.ff.experts.{e}.down_proj.weight"])
    x = x + y
    # layer 1: rotary positions, dense feed-forward, mixer and feed-forward in parallel on one norm
    h = P.rms_norm(x, w["t.1.n1"], 1e-5)
    q, k, v = qkv(1, h)
    f = P.rope_inv_freq(D, 10000.0, None)
    a = P.attention(P.apply_rope(q, pos, f), P.apply_rope(k, pos, f), v).reshape(T, NH * D) @ w["t.1.mix.o_proj.weight"].double().T
    x = x + a + P.gated_mlp(h, w["t.1.ff.gate_proj.weight"], w["t.1.ff.up_proj.weight"], w["t.1.ff.down_proj.weight"])
    return P.rms_norm(x, w["t.norm"], 1e-5) @ w["t.embed"].double().T


def test_toy_feed_forward_position_encoding_and_block(tmp_path, cuda_device):
    from gollmgo_b200.config import EngineConfig, register_architecture
    from gollmgo_b200.engine.batch import StepEntry
    from gollmgo_b200.engine.runner import load_runner
    from gollmgo_b200.parts import register_block, register_feed_forward, register_position
    from gollmgo_b200.weights import write_random_model
    register_feed_forward("toy_routed", RoutedFeedForward)
    register_position("toy_learned_scale", LearnedScalePositions)
    register_block("toy_parallel", ParallelBlock)
    register_architecture("ToyPartsForCausalLM", lambda d: d, toy_spec)
    cfg = {"architectures": ["ToyPartsForCausalLM"]}
    d = write_random_model(str(tmp_path / "toy"), cfg, seed=5, dtype="float32", std=0.2, norm_jitter=0.1)
    w = {k: v.float() for k, v in load_file(os.path.join(d, "model.safetensors")).items()}
    assert "t.0.ff.experts.1.down_proj.weight" in w and "t.1.n2" in w      # an unused norm is still a tensor of the layer
    runner = load_runner(d, EngineConfig(dtype="float32", block_size=8, num_blocks=32, max_batch_size=4,
                                         max_token_budget=128, cuda_graphs=False))
    g = torch.Generator().manual_seed(1)
    a = torch.randint(0, V, (37,), generator=g).tolist()
    b = torch.randint(0, V, (20,), generator=g).tolist()
    ref_a, ref_b = plain(w, a), plain(w, b)
    got = runner.step([StepEntry("a", a, range(37))]).cpu().double()
    torch.testing.assert_close(got, ref_a, rtol=2e-4, atol=2e-4)
    runner.release("a")
    rows = {"a": [], "b": []}
    for step in ([("a", 0, 10), ("b", 0, 2)], [("a", 10, 11), ("b", 2, 19)], [("a", 11, 36), ("b", 19, 20)], [("a", 36, 37)]):
        out = runner.step([StepEntry(r, {"a": a, "b": b}[r][lo:hi], range(hi - lo)) for r, lo, hi in step]).cpu().double()
        i = 0
        for r, lo, hi in step:
            rows[r].append(out[i:i + hi - lo])
            i += hi - lo
    torch.testing.assert_close(torch.cat(rows["a"]), ref_a, rtol=2e-4, atol=2e-4)
    torch.testing.assert_close(torch.cat(rows["b"]), ref_b, rtol=2e-4, atol=2e-4)
    runner.release("a"), runner.release("b")
    runner.cache.audit()


class LearnedPositionTable:
    """A learned vector per absolute position, added to the embedded tokens before the first layer."""
    interleaved = False

    def __init__(self, spec, ctx):
        self.max_pos, self.hidden = int(spec["max_positions"]), int(spec["hidden_size"])
        self.table = None

    def rope_table(self):
        return None

    def weights(self):
        from gollmgo_b200.weights import WeightSpec
        return {"table": WeightSpec((self.max_pos, self.hidden))}

    def load(self, get):
        self.table = get("table").float()

    def add_to_embedding(self, resid, batch):
        T = resid.shape[0]
        resid += self.table[batch.positions[:T].long()]


def learned_positions_spec(cfg):
    """One attention layer with no position encoding of its own; positions enter at the embedding."""
    from gollmgo_b200.parts import LayerSpec, ModelSpec, PartSpec, RunEntry
    norm = PartSpec("rmsnorm", {"size": H, "eps": 1e-5})
    attn = PartSpec("attention", {"hidden_size": H, "num_heads": NH, "num_kv_heads": NKV, "head_dim": D,
                                  "window": None, "position": PartSpec("none")})
    layer = LayerSpec(PartSpec("pre_norm"), attn, PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": I}),
                      norm, norm, mixer_prefix="l.mix.", ffn_prefix="l.ff.", mixer_norm_name="l.n1", ffn_norm_name="l.n2")
    return ModelSpec("LearnedPosForCausalLM", V, H, (layer,), (RunEntry(0, 0),), norm, True, "l.embed", "l.norm",
                     "l.head", MAXPOS,
                     embed_position=PartSpec("toy_learned_table", {"max_positions": MAXPOS, "hidden_size": H}),
                     embed_position_prefix="l.pos.")


def test_a_position_encoding_at_the_embedding(tmp_path, cuda_device):
    """A position encoding that is no part of any mixer: named in the ModelSpec, it gets its tensors
    from the checkpoint and the step's positions from the batch, whole and in portions alike."""
    from gollmgo_b200.config import EngineConfig, register_architecture
    from gollmgo_b200.engine.batch import StepEntry
    from gollmgo_b200.engine.runner import load_runner
    from gollmgo_b200.parts import register_position
    from gollmgo_b200.weights import write_random_model
    register_position("toy_learned_table", LearnedPositionTable)
    register_architecture("LearnedPosForCausalLM", lambda d: d, learned_positions_spec)
    d = write_random_model(str(tmp_path / "lp"), {"architectures": ["LearnedPosForCausalLM"]}, seed=6,
                           dtype="float32", std=0.2, norm_jitter=0.1)
    w = {k: v.double() for k, v in load_file(os.path.join(d, "model.safetensors")).items()}
    assert tuple(w["l.pos.table"].shape) == (MAXPOS, H)
    g = torch.Generator().manual_seed(2)
    toks = torch.randint(0, V, (29,), generator=g).tolist()
    T = len(toks)
    x = P.embed(w["l.embed"], toks) + w["l.pos.table"][:T]
    h = P.rms_norm(x, w["l.n1"], 1e-5)
    q = (h @ w["l.mix.q_proj.weight"].T).view(T, NH, D)
    k = (h @ w["l.mix.k_proj.weight"].T).view(T, NKV, D)
    v = (h @ w["l.mix.v_proj.weight"].T).view(T, NKV, D)
    x = x + P.attention(q, k, v).reshape(T, NH * D) @ w["l.mix.o_proj.weight"].T
    x = x + P.gated_mlp(P.rms_norm(x, w["l.n2"], 1e-5), w["l.ff.gate_proj.weight"], w["l.ff.up_proj.weight"],
                        w["l.ff.down_proj.weight"])
    want = P.rms_norm(x, w["l.norm"], 1e-5) @ w["l.embed"].T
    runner = load_runner(d, EngineConfig(dtype="float32", block_size=8, num_blocks=16, max_batch_size=2,
                                         max_token_budget=64))
    got = runner.step([StepEntry("w", toks, range(T))]).cpu().double()
    torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-4)
    rows = []
    for lo, hi in ((0, 11), (11, 13), (13, 28), (28, 29)):
        rows.append(runner.step([StepEntry("c", toks[lo:hi], range(hi - lo))]).cpu().double())
    torch.testing.assert_close(torch.cat(rows), want, rtol=2e-4, atol=2e-4)
    runner.release("w"), runner.release("c")
    runner.cache.audit()
