"""A toy mixer with state of its own, and a toy architecture that uses it, defined
HERE and registered without a change to the package: it is built from a config,
given random weights, stepped through the runner in portions and token by token,
and compared with a plain recurrence.  The toy run order also names a layer twice
and lets one layer read another layer's cache."""
import os

import pytest
import torch
from safetensors.torch import load_file

import plain_llama as P

pytestmark = pytest.mark.gpu

H, NH, NKV, D, I, V = 32, 4, 2, 16, 80, 97
DECAY = 0.75


class EmaMixer:
    """s_t = decay * s_{t-1} + (1 - decay) * x_t per request; y_t = s_t W^T.  The state
    is one float32 vector per request, kept in the request's state slot."""

    def __init__(self, spec, ctx):
        self.hidden, self.decay, self.ctx = int(spec["hidden_size"]), float(spec["decay"]), ctx
        self.w = None

    def cache_need(self):
        from gollmgo_b200.cache import FixedStateNeed
        return FixedStateNeed((self.hidden,), "float32")

    def weights(self):
        from gollmgo_b200.weights import WeightSpec
        return {"proj.weight": WeightSpec((self.hidden, self.hidden))}

    def load(self, get):
        self.w = get("proj.weight").float()

    def forward(self, x, batch, state, writes_cache=True):
        out = torch.empty_like(x)
        t = 0
        for slot, n, start in zip(batch.state_slot_list, batch.q_lens, batch.q_starts):
            s = state[slot]
            if start == 0:
                s.zero_()
            for i in range(n):
                s.mul_(self.decay).add_(x[t + i].float(), alpha=1 - self.decay)
                out[t + i] = (s @ self.w.T).to(x.dtype)
            t += n
        return out


def toy_spec(cfg):
    from gollmgo_b200.parts import LayerSpec, ModelSpec, PartSpec, RunEntry
    norm = PartSpec("rmsnorm", {"size": H, "eps": cfg["eps"]})
    ffn = PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": I})
    pos = PartSpec("rope", {"head_dim": D, "theta": 10000.0, "scaling": None})
    attn = PartSpec("attention", {"hidden_size": H, "num_heads": NH, "num_kv_heads": NKV, "head_dim": D,
                                  "window": None, "position": pos})
    ema = PartSpec("toy_ema", {"hidden_size": H, "decay": cfg["decay"]})

    def layer(i, mixer):
        return LayerSpec(PartSpec("pre_norm"), mixer, ffn, norm, norm, mixer_prefix=f"toy.{i}.mix.",
                         ffn_prefix=f"toy.{i}.ffn.", mixer_norm_name=f"toy.{i}.n1", ffn_norm_name=f"toy.{i}.n2")
    # layer 0 (attention) runs twice with a cache of its own each time; layer 1 keeps state;
    # layer 2 (attention) writes nothing and reads what the first run of layer 0 wrote
    order = (RunEntry(0, 0), RunEntry(1, 1), RunEntry(0, 2), RunEntry(2, 0, writes_cache=False))
    return ModelSpec("ToyForCausalLM", V, H, (layer(0, attn), layer(1, ema), layer(2, attn)), order, norm,
                     tie_embeddings=True, embed_name="toy.embed", final_norm_name="toy.norm",
                     head_name="toy.head", max_positions=512)


def plain_toy(w, cfg, toks):
    T = len(toks)
    x = P.embed(w["toy.embed"], toks)
    f = P.rope_inv_freq(D, 10000.0, None)
    pos = torch.arange(T)
    kv0 = {}

    def attn_layer(x, i, reuse=None):
        h = P.rms_norm(x, w[f"toy.{i}.n1"], cfg["eps"])
        q = P.apply_rope((h @ w[f"toy.{i}.mix.q_proj.weight"].double().T).view(T, NH, D), pos, f)
        if reuse is None:
            k = P.apply_rope((h @ w[f"toy.{i}.mix.k_proj.weight"].double().T).view(T, NKV, D), pos, f)
            v = (h @ w[f"toy.{i}.mix.v_proj.weight"].double().T).view(T, NKV, D)
        else:
            k, v = reuse
        x = x + P.attention(q, k, v).reshape(T, NH * D) @ w[f"toy.{i}.mix.o_proj.weight"].double().T
        h = P.rms_norm(x, w[f"toy.{i}.n2"], cfg["eps"])
        return x + P.gated_mlp(h, w[f"toy.{i}.ffn.gate_proj.weight"], w[f"toy.{i}.ffn.up_proj.weight"],
                               w[f"toy.{i}.ffn.down_proj.weight"]), (k, v)

    x, kv0 = attn_layer(x, 0)
    h = P.rms_norm(x, w["toy.1.n1"], cfg["eps"])
    s = torch.zeros(H, dtype=torch.float64)
    y = torch.empty_like(h)
    for t in range(T):
        s = cfg["decay"] * s + (1 - cfg["decay"]) * h[t]
        y[t] = s @ w["toy.1.mix.proj.weight"].double().T
    x = x + y
    h = P.rms_norm(x, w["toy.1.n2"], cfg["eps"])
    x = x + P.gated_mlp(h, w["toy.1.ffn.gate_proj.weight"], w["toy.1.ffn.up_proj.weight"], w["toy.1.ffn.down_proj.weight"])
    x, _ = attn_layer(x, 0)
    x, _ = attn_layer(x, 2, reuse=kv0)
    return P.rms_norm(x, w["toy.norm"], cfg["eps"]) @ w["toy.embed"].double().T


def test_toy_mixer_registers_builds_and_steps(tmp_path, cuda_device):
    from gollmgo_b200.config import EngineConfig, register_architecture
    from gollmgo_b200.engine.batch import StepEntry
    from gollmgo_b200.engine.runner import load_runner
    from gollmgo_b200.parts import register_mixer
    from gollmgo_b200.weights import write_random_model
    register_mixer("toy_ema", EmaMixer)
    register_architecture("ToyForCausalLM", lambda d: d, toy_spec)
    cfg = {"architectures": ["ToyForCausalLM"], "eps": 1e-5, "decay": DECAY}
    d = write_random_model(str(tmp_path / "toy"), cfg, seed=2, dtype="float32", std=0.15, norm_jitter=0.1)
    w = {k: v.float() for k, v in load_file(os.path.join(d, "model.safetensors")).items()}
    assert "toy.1.mix.proj.weight" in w and "toy.2.mix.k_proj.weight" in w and "toy.head" not in w
    runner = load_runner(d, EngineConfig(dtype="float32", block_size=8, num_blocks=32, max_batch_size=4,
                                         max_token_budget=128, cuda_graphs=False))
    assert len(runner.cache.groups) == 1 and sorted(runner.cache.group_of) == [0, 2]
    assert list(runner.cache.state_needs) == [1]
    g = torch.Generator().manual_seed(0)
    a = torch.randint(0, V, (41,), generator=g).tolist()
    b = torch.randint(0, V, (23,), generator=g).tolist()
    ref_a, ref_b = plain_toy(w, cfg, a), plain_toy(w, cfg, b)
    # whole
    got = runner.step([StepEntry("a", a, range(41))]).cpu().double()
    torch.testing.assert_close(got, ref_a, rtol=2e-4, atol=2e-4)
    runner.release("a")
    # a in portions and then token by token, b beside it; state and cache carry over between steps
    rows = {"a": [], "b": []}
    plan = [[("a", 0, 9), ("b", 0, 2)], [("a", 9, 20)], [("b", 2, 17), ("a", 20, 21)], [("a", 21, 22), ("b", 17, 18)],
            [("a", 22, 40), ("b", 18, 23)], [("a", 40, 41)]]
    for step in plan:
        entries = [StepEntry(r, {"a": a, "b": b}[r][lo:hi], range(hi - lo)) for r, lo, hi in step]
        out = runner.step(entries).cpu().double()
        i = 0
        for r, lo, hi in step:
            rows[r].append(out[i:i + hi - lo])
            i += hi - lo
    torch.testing.assert_close(torch.cat(rows["a"]), ref_a, rtol=2e-4, atol=2e-4)
    torch.testing.assert_close(torch.cat(rows["b"]), ref_b, rtol=2e-4, atol=2e-4)
    runner.release("a"), runner.release("b")
    runner.cache.audit()
    assert runner.cache.slots.num_free == runner.cache.slots.max_requests


class TileProbeMixer:
    """A mixer without cache or state that asks the batch builder for an index list of its own
    (tiles of 32 query rows, those with most keys first) and tags steps of three or more
    sequences.  It records what it is given; y = x W^T."""
    seen = []

    def __init__(self, spec, ctx):
        from gollmgo_b200.parts import QueryTiles
        self.hidden = int(spec["hidden_size"])
        self.need = QueryTiles(32, most_keys_first=True)
        self.w = None

    def cache_need(self):
        return None

    def query_tiles(self):
        return [self.need]

    def step_tags(self, facts):
        return ("crowd",) if facts.num_seqs >= 3 else ()

    def weights(self):
        from gollmgo_b200.weights import WeightSpec
        return {"proj.weight": WeightSpec((self.hidden, self.hidden))}

    def load(self, get):
        self.w = get("proj.weight").float()

    def forward(self, x, batch, cache, writes_cache=True):
        tl = batch.tiles[self.need]
        TileProbeMixer.seen.append((list(zip(tl.seq[:tl.count].tolist(), tl.q0[:tl.count].tolist())) if tl.count else [],
                                    batch.tags, batch.num_portions, sorted(k.height for k in batch.tiles)))
        return (x.float() @ self.w.T).to(x.dtype)


def probe_spec(cfg):
    from gollmgo_b200.parts import LayerSpec, ModelSpec, PartSpec, RunEntry
    norm = PartSpec("rmsnorm", {"size": H, "eps": 1e-5})
    ffn = PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": I})
    layer = LayerSpec(PartSpec("pre_norm"), PartSpec("toy_tile_probe", {"hidden_size": H}), ffn, norm, norm,
                      mixer_prefix="p.mix.", ffn_prefix="p.ffn.", mixer_norm_name="p.n1", ffn_norm_name="p.n2")
    return ModelSpec("ProbeForCausalLM", V, H, (layer,), (RunEntry(0, 0),), norm, tie_embeddings=True,
                     embed_name="p.embed", final_norm_name="p.norm", head_name="p.head", max_positions=512)


def test_a_mixer_gets_the_index_lists_and_step_tags_it_declares(tmp_path, cuda_device):
    """The batch builder builds exactly the lists the model's mixers ask for (here one list of
    32-row tiles and nothing of the attention kernels'), and the runner keys its captured
    steps by the tags the parts give, without knowing either."""
    from gollmgo_b200.config import EngineConfig, register_architecture
    from gollmgo_b200.engine.batch import StepEntry
    from gollmgo_b200.engine.runner import load_runner
    from gollmgo_b200.parts import register_mixer
    from gollmgo_b200.weights import write_random_model
    register_mixer("toy_tile_probe", TileProbeMixer)
    register_architecture("ProbeForCausalLM", lambda d: d, probe_spec)
    d = write_random_model(str(tmp_path / "probe"), {"architectures": ["ProbeForCausalLM"]}, seed=4, dtype="float32",
                           std=0.2)
    w = {k: v.double() for k, v in load_file(os.path.join(d, "model.safetensors")).items()}
    runner = load_runner(d, EngineConfig(dtype="float32", block_size=8, num_blocks=8, max_batch_size=4,
                                         max_token_budget=256))
    assert not runner.cache.groups                                   # nothing is paged for this model
    TileProbeMixer.seen.clear()
    g = torch.Generator().manual_seed(1)
    toks = {r: torch.randint(0, V, (n,), generator=g).tolist() for r, n in (("a", 70), ("b", 1), ("c", 33))}
    out = runner.step([StepEntry(r, t, [len(t) - 1]) for r, t in toks.items()]).cpu().double()
    tiles, tags, portions, heights = TileProbeMixer.seen[-1]
    assert heights == [32] and portions == 2 and tags == ("crowd",)
    assert tiles == [(0, 64), (0, 32), (2, 32), (0, 0), (2, 0)]      # most keys first; the single token has no tile
    # the model is position-free: every row is a function of its own token
    def plain(t):
        x = P.embed(w["p.embed"], [t])
        x = x + P.rms_norm(x, w["p.n1"], 1e-5) @ w["p.mix.proj.weight"].T
        x = x + P.gated_mlp(P.rms_norm(x, w["p.n2"], 1e-5), w["p.ffn.gate_proj.weight"], w["p.ffn.up_proj.weight"],
                            w["p.ffn.down_proj.weight"])
        return (P.rms_norm(x, w["p.norm"], 1e-5) @ w["p.embed"].T)[0]
    for i, r in enumerate(toks):
        torch.testing.assert_close(out[i], plain(toks[r][-1]), rtol=2e-4, atol=2e-4)
    # decode-only steps: captured per (bucket, tags)
    TileProbeMixer.seen.clear()
    runner.step([StepEntry(r, [5], [0]) for r in ("a", "b", "c")])
    runner.step([StepEntry(r, [6], [0]) for r in ("a", "b")])
    assert (4, ("crowd",)) in runner._graphs and 2 in runner._graphs
    assert {s[1] for s in TileProbeMixer.seen} == {("crowd",), ()} and all(s[0] == [] for s in TileProbeMixer.seen)
    for r in toks:
        runner.release(r)
    runner.cache.audit()
