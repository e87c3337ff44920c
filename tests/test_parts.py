"""Each part of the model alone (norm, position encoding, mixer, feed-forward, block)
against the plain implementation's function for that part, in float32 and bfloat16,
at sizes that are none of the tiny configurations'."""
import math

import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu


def close(got, want, dtype):
    """Worst error relative to the size of the result: float32 keeps 1e-5, bfloat16
    (8 bits of mantissa, a few roundings in a row) 2e-2."""
    err = float((got - want).abs().max() / want.abs().max())
    assert err <= (1e-5 if dtype == torch.float32 else 2e-2), f"relative error {err:.2e}"


@pytest.fixture(scope="module")
def kit(cuda_device):
    from gollmgo_b200 import parts
    from gollmgo_b200.cache import CacheManager
    from gollmgo_b200.engine.batch import BatchBuilder, StepEntry
    parts.set_matmul_precision()

    class Kit:
        pass
    k = Kit()
    k.parts, k.CacheManager, k.BatchBuilder, k.StepEntry = parts, CacheManager, BatchBuilder, StepEntry
    return k


def ctx_for(kit, dtype, page=16):
    return kit.parts.BuildContext(dtype, "cuda", max_tokens=256, max_seqs=8, page_size=page)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(kit, dtype):
    ctx = ctx_for(kit, dtype)
    n = kit.parts.build_norm(kit.parts.PartSpec("rmsnorm", {"size": 72, "eps": 2e-6}), ctx)
    w = 1 + 0.2 * torch.randn(72)
    n.load(lambda name: w.cuda().to(dtype))
    assert n.weights()[""].shape == (72,)
    resid = torch.randn(5, 72, device="cuda")
    delta = torch.randn(5, 72, device="cuda").to(dtype)
    want = P.rms_norm(resid.cpu().double() + delta.cpu().double(), w.to(dtype), 2e-6)
    out = torch.empty(5, 72, device="cuda", dtype=dtype)
    n.add_norm(resid, delta, out)
    close(out.cpu().double(), want, dtype)


def test_position_part_tables(kit):
    from gollmgo_b200.config import RopeScaling
    ctx = ctx_for(kit, torch.float32)
    sc = {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 2.0,
          "original_max_position_embeddings": 32}
    rope = kit.parts.build_position(kit.parts.PartSpec("rope", {
        "head_dim": 48, "theta": 12345.0, "scaling": RopeScaling("llama3", 4.0, 1.0, 2.0, 32)}), ctx)
    torch.testing.assert_close(rope.rope_table().cpu(), P.rope_inv_freq(48, 12345.0, sc), rtol=1e-13, atol=0)
    lin = kit.parts.build_position(kit.parts.PartSpec("rope", {
        "head_dim": 16, "theta": 10000.0, "scaling": RopeScaling("linear", 2.0)}), ctx)
    torch.testing.assert_close(lin.rope_table().cpu(), P.rope_inv_freq(16, 10000.0, {"rope_type": "linear", "factor": 2.0}), rtol=1e-13, atol=0)
    assert kit.parts.build_position(kit.parts.PartSpec("none"), ctx).rope_table() is None
    with pytest.raises(KeyError, match="known"):
        kit.parts.build_position(kit.parts.PartSpec("alibi"), ctx)


def run_mixer(kit, mixer, need, x_parts, dtype, page):
    """Step the mixer over one sequence cut into the given portions; return all outputs."""
    cm = kit.CacheManager([need], page, 64, 4, dtype=dtype, device="cuda")
    bb = kit.BatchBuilder(cm, "cuda", query_tiles=getattr(mixer, "query_tiles", lambda: ())())
    cm.admit("s")
    outs = []
    for x in x_parts:
        batch = bb.build([kit.StepEntry("s", [0] * x.shape[0], [])])
        outs.append(mixer.forward(x.cuda().to(dtype).contiguous(), batch, cm.layer_cache(0)).clone())
    return torch.cat(outs).cpu().double()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d,window,interleaved,page", [(6, 2, 16, None, False, 16), (3, 3, 32, 9, True, 8)])
def test_attention_mixer(kit, dtype, nh, nkv, d, window, interleaved, page):
    torch.manual_seed(0)
    H, T = 40, 45
    ctx = ctx_for(kit, dtype, page)
    pos = kit.parts.PartSpec("rope", {"head_dim": d, "theta": 777.0, "scaling": None, "interleaved": interleaved})
    mixer = kit.parts.build_mixer(kit.parts.PartSpec("attention", {
        "hidden_size": H, "num_heads": nh, "num_kv_heads": nkv, "head_dim": d, "window": window,
        "position": pos}), ctx)
    w = {n: (torch.randn(s.shape) * 0.3).to(dtype) for n, s in mixer.weights().items()}
    mixer.load(lambda n: w[n].cuda())
    need = mixer.cache_need()
    assert (need.n_kv_heads, need.head_dim, need.window) == (nkv, d, window)
    x = torch.randn(T, H).to(dtype)
    # plain: project, rotate, attend, project
    xd = x.double()
    q = (xd @ w["q_proj.weight"].double().T).view(T, nh, d)
    k = (xd @ w["k_proj.weight"].double().T).view(T, nkv, d)
    v = (xd @ w["v_proj.weight"].double().T).view(T, nkv, d)
    f = P.rope_inv_freq(d, 777.0, None)
    q, k = P.apply_rope(q, torch.arange(T), f, interleaved), P.apply_rope(k, torch.arange(T), f, interleaved)
    want = P.attention(q, k, v, window).reshape(T, nh * d) @ w["o_proj.weight"].double().T
    whole = run_mixer(kit, mixer, need, [x], dtype, page)
    cut = run_mixer(kit, mixer, need, [x[:7], x[7:9], x[9:30], x[30:31], x[31:]], dtype, page)
    close(whole, want, dtype)
    close(cut, want, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(kit, dtype):
    torch.manual_seed(1)
    H, I, T = 56, 150, 9
    ctx = ctx_for(kit, dtype)
    ff = kit.parts.build_feed_forward(kit.parts.PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": I}), ctx)
    w = {n: (torch.randn(s.shape) * 0.3).to(dtype) for n, s in ff.weights().items()}
    ff.load(lambda n: w[n].cuda())
    x = torch.randn(T, H).to(dtype)
    got = ff.forward(x.cuda(), None).cpu().double()
    want = P.gated_mlp(x, w["gate_proj.weight"], w["up_proj.weight"], w["down_proj.weight"])
    close(got, want, dtype)
    with pytest.raises(ValueError, match="activation"):
        kit.parts.build_feed_forward(kit.parts.PartSpec("gated_mlp", {"hidden_size": 8, "intermediate_size": 8, "activation": "relu"}), ctx)


def test_weight_stored_in_float32_is_multiplied_in_float32(kit):
    """bfloat16 activations with a float32 weight: the product is a float32 one."""
    torch.manual_seed(2)
    x = torch.randn(4, 64, device="cuda").to(torch.bfloat16)
    w = torch.randn(24, 64, device="cuda")
    out = torch.empty(4, 24, device="cuda", dtype=torch.bfloat16)
    kit.parts.linear(x, w, out)
    want = (x.float() @ w.T).to(torch.bfloat16)
    assert torch.equal(out, want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_is_the_plain_decoder_layer(kit, dtype):
    torch.manual_seed(3)
    cfg = {"hidden_size": 48, "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 16,
           "intermediate_size": 100, "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "num_hidden_layers": 1}
    ctx = ctx_for(kit, dtype)
    S = kit.parts.PartSpec
    pos = S("rope", {"head_dim": 16, "theta": 10000.0, "scaling": None})
    mixer = kit.parts.build_mixer(S("attention", {"hidden_size": 48, "num_heads": 3, "num_kv_heads": 1,
                                                  "head_dim": 16, "window": None, "position": pos}), ctx)
    ff = kit.parts.build_feed_forward(S("gated_mlp", {"hidden_size": 48, "intermediate_size": 100}), ctx)
    n1 = kit.parts.build_norm(S("rmsnorm", {"size": 48, "eps": 1e-5}), ctx)
    n2 = kit.parts.build_norm(S("rmsnorm", {"size": 48, "eps": 1e-5}), ctx)
    layer = kit.parts.LayerSpec(S("pre_norm"), None, None, None, None)
    block = kit.parts.build_block(layer, mixer, ff, n1, n2, ctx)
    p = "model.layers.0."
    w = {}
    for pre, part in ((p + "self_attn.", mixer), (p + "mlp.", ff)):
        for n, s in part.weights().items():
            w[pre + n] = (torch.randn(s.shape) * 0.2).to(dtype)
    w[p + "input_layernorm.weight"] = (1 + 0.1 * torch.randn(48)).to(dtype)
    w[p + "post_attention_layernorm.weight"] = (1 + 0.1 * torch.randn(48)).to(dtype)
    mixer.load(lambda n: w[p + "self_attn." + n].cuda())
    ff.load(lambda n: w[p + "mlp." + n].cuda())
    n1.load(lambda n: w[p + "input_layernorm.weight"].cuda())
    n2.load(lambda n: w[p + "post_attention_layernorm.weight"].cuda())
    T = 21
    x0 = torch.randn(T, 48)
    want = P.decoder_layer(x0.double(), w, 0, cfg, torch.arange(T), P.rope_inv_freq(16, 10000.0, None), None)
    cm = kit.CacheManager([mixer.cache_need()], 16, 16, 2, dtype=dtype, device="cuda")
    bb = kit.BatchBuilder(cm, "cuda", query_tiles=mixer.query_tiles())
    cm.admit("s")
    batch = bb.build([kit.StepEntry("s", [0] * T, [])])
    resid = x0.cuda().clone()
    delta = block.forward(resid, None, batch, cm.layer_cache(0))
    got = resid.cpu().double() + delta.cpu().double()            # the block still owes its last delta
    close(got, want, dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("fuse", [True, False])
def test_two_blocks_of_a_short_step_with_norms_inside_the_products(kit, cuda_device, monkeypatch, fuse):
    """Steps of up to 16 tokens in bfloat16: the residual adds and norms between the products
    are done by the products (parts/linear.py).  Two chained blocks give the plain result
    either way, and the fused way really hands NormedRows from block to block."""
    import importlib
    L = importlib.import_module("gollmgo_b200.parts.linear")     # the package also exports a function of that name
    monkeypatch.setattr(L, "FUSE_NORMS", fuse)
    dtype = torch.bfloat16
    torch.manual_seed(11)
    Hd, nh, nkv, d, I = 64, 4, 2, 16, 104
    cfg = {"hidden_size": Hd, "num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": d,
           "intermediate_size": I, "rms_norm_eps": 2e-6, "rope_theta": 10000.0, "num_hidden_layers": 2}
    ctx = ctx_for(kit, dtype)
    S = kit.parts.PartSpec
    pos = S("rope", {"head_dim": d, "theta": 10000.0, "scaling": None})
    blocks, w = [], {}
    for l in range(2):
        mixer = kit.parts.build_mixer(S("attention", {"hidden_size": Hd, "num_heads": nh, "num_kv_heads": nkv,
                                                      "head_dim": d, "window": None, "position": pos}), ctx)
        ff = kit.parts.build_feed_forward(S("gated_mlp", {"hidden_size": Hd, "intermediate_size": I}), ctx)
        n1 = kit.parts.build_norm(S("rmsnorm", {"size": Hd, "eps": 2e-6}), ctx)
        n2 = kit.parts.build_norm(S("rmsnorm", {"size": Hd, "eps": 2e-6}), ctx)
        p = f"model.layers.{l}."
        for pre, part in ((p + "self_attn.", mixer), (p + "mlp.", ff)):
            for n, s in part.weights().items():
                w[pre + n] = (torch.randn(s.shape) * 0.2).to(dtype)
        w[p + "input_layernorm.weight"] = (1 + 0.1 * torch.randn(Hd)).to(dtype)
        w[p + "post_attention_layernorm.weight"] = (1 + 0.1 * torch.randn(Hd)).to(dtype)
        mixer.load(lambda n, p=p: w[p + "self_attn." + n].cuda())
        ff.load(lambda n, p=p: w[p + "mlp." + n].cuda())
        n1.load(lambda n, p=p: w[p + "input_layernorm.weight"].cuda())
        n2.load(lambda n, p=p: w[p + "post_attention_layernorm.weight"].cuda())
        blocks.append((kit.parts.build_block(kit.parts.LayerSpec(S("pre_norm"), None, None, None, None),
                                             mixer, ff, n1, n2, ctx), mixer))
    T = 7                                                            # one portion of 7 tokens
    x0 = torch.randn(T, Hd)
    inv = P.rope_inv_freq(d, 10000.0, None)
    want = x0.double()
    for l in range(2):
        want = P.decoder_layer(want, w, l, cfg, torch.arange(T), inv, None)
    cm = kit.CacheManager([blocks[0][1].cache_need(), blocks[1][1].cache_need()], 16, 16, 2, dtype=dtype, device="cuda")
    bb = kit.BatchBuilder(cm, "cuda", query_tiles=blocks[0][1].query_tiles())
    cm.admit("s")
    batch = bb.build([kit.StepEntry("s", [0] * T, [])])
    resid = x0.cuda().clone()
    d0 = blocks[0][0].forward(resid, None, batch, cm.layer_cache(0), next_block=blocks[1][0])
    assert isinstance(d0, L.NormedRows) == fuse
    d1 = blocks[1][0].forward(resid, d0, batch, cm.layer_cache(1), next_block=None)
    assert isinstance(d1, torch.Tensor)                              # nothing runs next: a plain delta
    got = resid.cpu().double() + d1.cpu().double()
    close(got, want, dtype)
