"""Each CUDA kernel alone against a plain float32 PyTorch reference of the same op,
at sizes other than the engine's: widths and vocabularies that are no power of
two, head sizes in steps of 16, ragged batches, permuted pages, contexts that
straddle page, tile and slice edges, and inputs made so that one far key decides
the result."""
import math
import random

import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


@pytest.fixture(scope="module")
def ops(cuda_device):
    from gollmgo_b200.csrc import ops as o
    assert o.device_capability() >= 100
    return o


# ---------------------------------------------------------------- embedding
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("V,H", [(301, 120), (1000, 4100)])
def test_embed_gather(ops, cuda_device, dtype, V, H):
    g = torch.Generator(device="cuda").manual_seed(0)
    table = torch.randn(V, H, device="cuda", generator=g).to(dtype)
    ids = torch.tensor([0, V - 1, 5, 5, 17, V // 2], dtype=torch.int32, device="cuda")
    out = torch.full((ids.numel(), H), 7.0, device="cuda")
    bad = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.embed_gather(ids, table, out, bad)
    assert torch.equal(out, table[ids.long()].float()) and int(bad) == 0


# ---------------------------------------------------------------- add + rmsnorm
def ref_rmsnorm(x, w, eps):
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,eps", [(100, 1e-5), (4096, 1e-6), (5120 + 16, 3e-6)])
def test_add_rmsnorm(ops, cuda_device, dtype, H, eps):
    g = torch.Generator(device="cuda").manual_seed(1)
    n = 7
    resid = torch.randn(n, H, device="cuda", generator=g) * 3
    delta = torch.randn(n, H, device="cuda", generator=g).to(dtype)
    w = 1 + 0.1 * torch.randn(H, device="cuda", generator=g)
    r0 = resid.clone()
    out = torch.empty(n, H, device="cuda", dtype=dtype)
    ops.add_rmsnorm(resid, delta, w, out, eps)
    x = r0 + delta.float()
    assert torch.equal(resid, x)                                       # the residual sum is float32, exact
    torch.testing.assert_close(out.float(), ref_rmsnorm(x, w, eps).to(dtype).float(), **tol(dtype))
    # no delta: the residual is left alone
    r1 = resid.clone()
    ops.add_rmsnorm(resid, None, w, out, eps)
    assert torch.equal(resid, r1)
    torch.testing.assert_close(out.float(), ref_rmsnorm(r1, w, eps).to(dtype).float(), **tol(dtype))
    # chosen rows, nothing written back
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device="cuda")
    out3 = torch.empty(3, H, device="cuda", dtype=dtype)
    ops.add_rmsnorm(resid, delta, w, out3, eps, rows=rows, write_back=False)
    assert torch.equal(resid, r1)
    torch.testing.assert_close(out3.float(), ref_rmsnorm(r1 + delta.float(), w, eps)[rows.long()].to(dtype).float(), **tol(dtype))


# ---------------------------------------------------------------- silu * up
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,I", [(1, 352), (5, 13), (33, 14336)])
def test_silu_mul(ops, cuda_device, dtype, T, I):
    g = torch.Generator(device="cuda").manual_seed(2)
    gu = (torch.randn(T, 2 * I, device="cuda", generator=g) * 3).to(dtype)
    out = torch.empty(T, I, device="cuda", dtype=dtype)
    ops.silu_mul(gu, out)
    gf, uf = gu[:, :I].float(), gu[:, I:].float()
    ref = (gf / (1 + torch.exp(-gf)) * uf).to(dtype)
    torch.testing.assert_close(out.float(), ref.float(), **tol(dtype))


# ---------------------------------------------------------------- rope + cache write
def ref_rope(x, pos, inv_freq, interleaved):
    """x [T, h, d] float64; rotates the first 2*len(inv_freq) elements of each head."""
    rot = 2 * inv_freq.numel()
    ang = pos.double()[:, None] * inv_freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    if interleaved:
        a, b = x[..., 0:rot:2], x[..., 1:rot:2]
        out[..., 0:rot:2], out[..., 1:rot:2] = a * c - b * s, a * s + b * c
    else:
        a, b = x[..., :rot // 2], x[..., rot // 2:rot]
        out[..., :rot // 2], out[..., rot // 2:rot] = a * c - b * s, a * s + b * c
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d,rot,interleaved,page", [
    (4, 2, 16, 16, False, 16), (5, 5, 48, 48, True, 8), (8, 1, 80, 32, False, 32), (3, 3, 128, 0, False, 16),
    (32, 8, 128, 128, False, 16), (6, 2, 64, 64, False, 8), (3, 1, 48, 48, False, 16)])
def test_rope_kv_write(ops, cuda_device, dtype, nh, nkv, d, rot, interleaved, page):
    g = torch.Generator(device="cuda").manual_seed(3)
    T, pages = 11, 9
    qkv = torch.randn(T, (nh + 2 * nkv) * d, device="cuda", generator=g).to(dtype)
    pos = torch.tensor([0, 1, 2, 70, 71, 500, 3, 9000, 4, 5, 6], dtype=torch.int32, device="cuda")
    slots = random.Random(0).sample(range(pages * page), T)
    slots[4] = -1                                                      # a token that is not to be written
    slot_t = torch.tensor(slots, dtype=torch.int32, device="cuda")
    inv = (1.0 / (10000.0 ** (torch.arange(0, rot, 2, dtype=torch.float64) / max(rot, 1)))).cuda() if rot else None
    kc = torch.full((pages, nkv, page, d), 9.0, device="cuda", dtype=dtype)
    vc = torch.full((pages, nkv, page, d), 9.0, device="cuda", dtype=dtype)
    x = qkv.clone()
    ops.rope_kv_write(x, pos, slot_t, inv, kc, vc, nh, nkv, d, page, interleaved, True)
    src = qkv.double().view(T, nh + 2 * nkv, d)
    qk = ref_rope(src[:, :nh + nkv], pos, inv, interleaved) if rot else src[:, :nh + nkv]
    got = x.double().view(T, nh + 2 * nkv, d)
    t = dict(rtol=1e-6, atol=1e-6) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(got[:, :nh + nkv], qk.to(dtype).double(), **t)
    assert torch.equal(got[:, nh + nkv:], src[:, nh + nkv:])           # v is untouched in place
    for i, s in enumerate(slots):
        if s < 0:
            continue
        p, o = divmod(s, page)
        assert torch.equal(kc[p, :, o], x.view(T, nh + 2 * nkv, d)[i, nh:nh + nkv])    # the rotated k
        assert torch.equal(vc[p, :, o], qkv.view(T, nh + 2 * nkv, d)[i, nh + nkv:])
    written = torch.zeros(pages * page, dtype=torch.bool)
    written[[s for s in slots if s >= 0]] = True
    flat = kc.permute(0, 2, 1, 3).reshape(pages * page, nkv, d)
    assert (flat[~written.cuda()] == 9.0).all()                        # nothing else was written


# ---------------------------------------------------------------- attention over the paged cache
def paged(seqs_kv, page, pages, nkv, d, dtype, seed):
    """Put each sequence's keys and values into randomly chosen pages.  Returns caches
    and block tables."""
    rng = random.Random(seed)
    free = list(range(pages))
    rng.shuffle(free)
    # everywhere else (pages nobody holds, a last page's rows past the context): NaN, which
    # reaches the output through any product, a zero probability's too
    kc = torch.full((pages, nkv, page, d), float("nan"), device="cuda", dtype=dtype)
    vc = torch.full((pages, nkv, page, d), float("nan"), device="cuda", dtype=dtype)
    stride = max(-(-k.shape[0] // page) for k, _ in seqs_kv) + 2
    bt = torch.full((len(seqs_kv), stride), -1, dtype=torch.int32)
    for b, (k, v) in enumerate(seqs_kv):
        for lp in range(-(-k.shape[0] // page)):
            pg = free.pop()
            bt[b, lp] = pg
            n = min(page, k.shape[0] - lp * page)
            kc[pg, :, :n] = k[lp * page:lp * page + n].transpose(0, 1)
            vc[pg, :, :n] = v[lp * page:lp * page + n].transpose(0, 1)
    return kc, vc, bt.cuda(), stride


def ref_attention(q, k, v, q_start, window):
    """q [n, nh, d] at positions q_start.., k/v [ctx, nkv, d] -> [n, nh, d] in float64."""
    n, nh, d = q.shape
    ctx, nkv, _ = k.shape
    qi = torch.arange(q_start, q_start + n, device=q.device)[:, None]
    kj = torch.arange(ctx, device=q.device)[None, :]
    ok = kj <= qi
    if window:
        ok &= kj > qi - window
    out = torch.empty(n, nh, d, dtype=torch.float64, device=q.device)
    for h in range(nh):
        s = q[:, h].double() @ k[:, h // (nh // nkv)].double().T / math.sqrt(d)
        p = torch.softmax(s.masked_fill(~ok, float("-inf")), dim=-1)
        out[:, h] = p @ v[:, h // (nh // nkv)].double()
    return out


def spike(q, k, v, head, nkv_of_head, key_pos, strength=30.0):
    """Make query `head` of the last token look almost only at key `key_pos`."""
    d = q.shape[-1]
    u = torch.randn(d, device=q.device)
    u /= u.norm()
    q[-1, head] = u * strength
    k[key_pos, nkv_of_head] = u * strength
    v[key_pos, nkv_of_head] = torch.arange(d, device=q.device).float() / d + 3.0


@pytest.mark.parametrize("allow_mma", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d,page,window", [
    (4, 2, 16, 16, 0), (4, 1, 32, 8, 0), (5, 5, 48, 32, 24), (32, 8, 128, 16, 0), (8, 2, 80, 16, 100),
    (2, 1, 256, 16, 0), (24, 1, 64, 16, 0), (6, 2, 64, 8, 70), (40, 2, 128, 32, 0), (3, 3, 128, 16, 33)])
def test_attn_decode(ops, cuda_device, dtype, nh, nkv, d, page, window, allow_mma):
    if allow_mma and not (dtype == torch.bfloat16 and d in (64, 128)):
        pytest.skip("the tensor-core kernel takes bfloat16 with head size 64 or 128")
    torch.manual_seed(4)
    ctxs = [1, 2, page - 1, page, page + 1, 63, 64, 65, 127, 129, 300, 777, 3000, 5001]
    B = len(ctxs)
    seqs, qs, refs = [], [], []
    for i, ctx in enumerate(ctxs):
        k, v = torch.randn(ctx, nkv, d, device="cuda"), torch.randn(ctx, nkv, d, device="cuda")
        q = torch.randn(1, nh, d, device="cuda")
        lo = max(0, ctx - window) if window else 0
        far = [lo, min(ctx - 1, lo + 1), ctx - 1, (lo + ctx) // 2, max(lo, ctx - 65)][i % 5]
        if ctx > 2000:
            far = lo + 3                                               # a key thousands of tokens back
        spike(q, k, v, i % nh, (i % nh) // (nh // nkv), far)
        q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
        seqs.append((k, v)), qs.append(q)
        refs.append(ref_attention(q.float(), k.float(), v.float(), ctx - 1, window))
    kc, vc, bt, stride = paged(seqs, page, sum(-(-c // page) for c in ctxs) + 5, nkv, d, dtype, 1)
    q_all = torch.cat(qs).reshape(B, nh * d).contiguous()
    cu = torch.arange(B + 1, dtype=torch.int32, device="cuda")
    ctx_t = torch.tensor(ctxs, dtype=torch.int32, device="cuda")
    order = list(range(B))
    random.Random(2).shuffle(order)
    dec = torch.tensor(order + [-1, -1], dtype=torch.int32, device="cuda")       # two padded entries
    for splits in (1, 3, 8, 11):                                       # up to 8 merge inside a cluster
        n_dec = B + 2
        part_o = torch.full((n_dec * nh * splits * d,), float("nan"), device="cuda")
        part_ml = torch.full((n_dec * nh * splits * 2,), float("nan"), device="cuda")
        out = torch.zeros(B, nh * d, device="cuda", dtype=dtype)
        ops.attn_decode(q_all, nh * d, kc, vc, bt, stride, cu, ctx_t, dec, n_dec, splits, part_o, part_ml,
                        out, nh, nkv, d, page, window, 1 / math.sqrt(d), allow_mma=allow_mma)
        ref = torch.cat(refs).reshape(B, nh * d)
        torch.testing.assert_close(out.double(), ref, **tol(dtype))


@pytest.mark.parametrize("nh,nkv,d,page,window", [
    (32, 8, 128, 16, 0), (24, 1, 64, 16, 0), (6, 2, 64, 8, 70), (40, 2, 128, 32, 0), (3, 3, 128, 16, 33)])
@pytest.mark.parametrize("many", [False, True])
def test_attn_decode_flat(ops, cuda_device, nh, nkv, d, page, window, many):
    """The decode kernel for large batches cuts the tiles of all (token, kv head) pairs into
    equal ranges, so a pair's keys may be spread over several CTAs and a CTA may hold the end
    of one pair and the start of the next: contexts from one key to thousands, padding
    entries in between, and (many) more pairs than CTAs."""
    dtype = torch.bfloat16
    torch.manual_seed(6)
    ctxs = [1, 2, page - 1, page, page + 1, 63, 64, 65, 127, 129, 300, 777, 3000, 5001]
    if many:
        ctxs = ctxs + [70 + 13 * i for i in range(150)]
    B = len(ctxs)
    seqs, qs, refs = [], [], []
    for i, ctx in enumerate(ctxs):
        k, v = torch.randn(ctx, nkv, d, device="cuda"), torch.randn(ctx, nkv, d, device="cuda")
        q = torch.randn(1, nh, d, device="cuda")
        lo = max(0, ctx - window) if window else 0
        far = [lo, min(ctx - 1, lo + 1), ctx - 1, (lo + ctx) // 2, max(lo, ctx - 65)][i % 5]
        if ctx > 2000:
            far = lo + 3
        spike(q, k, v, i % nh, (i % nh) // (nh // nkv), far)
        q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
        seqs.append((k, v)), qs.append(q)
        refs.append(ref_attention(q.float(), k.float(), v.float(), ctx - 1, window))
    kc, vc, bt, stride = paged(seqs, page, sum(-(-c // page) for c in ctxs) + 5, nkv, d, dtype, 1)
    q_all = torch.cat(qs).reshape(B, nh * d).contiguous()
    cu = torch.arange(B + 1, dtype=torch.int32, device="cuda")
    ctx_t = torch.tensor(ctxs, dtype=torch.int32, device="cuda")
    order = list(range(B))
    random.Random(2).shuffle(order)
    order[3:3] = [-1]                                                   # padding in the middle and at the end
    dec = torch.tensor(order + [-1, -1], dtype=torch.int32, device="cuda")
    n_dec = len(order) + 2
    pieces = ops.attn_decode_flat_pieces(n_dec, nh, nkv, d)
    part_o = torch.full((pieces * 16 * d,), float("nan"), device="cuda")
    part_ml = torch.full((pieces * 16 * 2,), float("nan"), device="cuda")
    prefix = torch.full((ops.attn_decode_flat_prefix_ints(n_dec, nh, nkv),), -7, dtype=torch.int32, device="cuda")
    out = torch.zeros(B, nh * d, device="cuda", dtype=dtype)
    ops.attn_decode_flat(q_all, nh * d, kc, vc, bt, stride, cu, ctx_t, dec, n_dec, part_o, part_ml, prefix,
                         out, nh, nkv, d, page, window, 1 / math.sqrt(d))
    ref = torch.cat(refs).reshape(B, nh * d)
    torch.testing.assert_close(out.double(), ref, **tol(dtype))
    # the same through the sliced kernel: equal up to the order of the sums
    out2 = torch.zeros_like(out)
    po = torch.empty(n_dec * nh * 3 * d, device="cuda")
    pm = torch.empty(n_dec * nh * 3 * 2, device="cuda")
    ops.attn_decode(q_all, nh * d, kc, vc, bt, stride, cu, ctx_t, dec, n_dec, 3, po, pm, out2,
                    nh, nkv, d, page, window, 1 / math.sqrt(d))
    torch.testing.assert_close(out.float(), out2.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("nh,nkv,d,page,window", [
    (32, 8, 128, 16, 0), (24, 2, 64, 16, 0), (6, 2, 64, 8, 70), (16, 1, 128, 32, 0), (3, 3, 128, 16, 33)])
def test_attn_decode_with_rotation_inside(ops, cuda_device, nh, nkv, d, page, window):
    """The decode kernel that rotates q and k and writes the cache itself gives, bit for bit,
    what rope_kv_write followed by attn_decode gives: outputs and cache."""
    dtype = torch.bfloat16
    torch.manual_seed(5)
    ctxs = [1, 2, page, page + 1, 64, 65, 128, 129, 300, 777, 3000]
    B = len(ctxs)
    seqs = [(torch.randn(c, nkv, d, device="cuda").to(dtype), torch.randn(c, nkv, d, device="cuda").to(dtype))
            for c in ctxs]
    kc, vc, bt, stride = paged(seqs, page, sum(-(-c // page) for c in ctxs) + 5, nkv, d, dtype, 7)
    W = (nh + 2 * nkv) * d
    qkv = torch.randn(B + 2, W, device="cuda").to(dtype)                  # two rows of padding at the end
    order = list(range(B))
    random.Random(3).shuffle(order)                                       # token t belongs to sequence order[t]
    cu = torch.zeros(B + 1, dtype=torch.int32)
    pos = torch.zeros(B + 2, dtype=torch.int32)
    slots = torch.full((B + 2,), -1, dtype=torch.int32)
    # sequence b has its one token in row t where order[t] == b; cu_q_lens is by sequence, so rows follow it
    rows = torch.empty(B + 2, W, device="cuda", dtype=dtype)
    for b in range(B):
        cu[b + 1] = b + 1
        pos[b] = ctxs[b] - 1
        slots[b] = int(bt[b, (ctxs[b] - 1) // page]) * page + (ctxs[b] - 1) % page
        rows[b] = qkv[b]
    rows[B:] = qkv[B:]
    cu, pos, slots = cu.cuda(), pos.cuda(), slots.cuda()
    ctx_t = torch.tensor(ctxs, dtype=torch.int32, device="cuda")
    dec = torch.tensor(order + [-1, -1], dtype=torch.int32, device="cuda")
    inv = (1.0 / (500000.0 ** (torch.arange(0, d, 2, dtype=torch.float64) / d))).cuda()
    for splits in (1, 4, 8, 11):
        n_dec = B + 2
        part_o = torch.empty(n_dec * nh * splits * d, device="cuda")
        part_ml = torch.empty(n_dec * nh * splits * 2, device="cuda")
        for write in (True, False):
            x1, k1, v1 = rows.clone(), kc.clone(), vc.clone()
            out1 = torch.zeros(B + 2, nh * d, device="cuda", dtype=dtype)
            ops.rope_kv_write(x1, pos, slots, inv, k1, v1, nh, nkv, d, page, False, write)
            ops.attn_decode(x1, W, k1, v1, bt, stride, cu, ctx_t, dec, n_dec, splits, part_o, part_ml, out1,
                            nh, nkv, d, page, window, 1 / math.sqrt(d))
            x2, k2, v2 = rows.clone(), kc.clone(), vc.clone()
            out2 = torch.zeros(B + 2, nh * d, device="cuda", dtype=dtype)
            ops.attn_decode_rope(x2, k2, v2, bt, stride, cu, ctx_t, dec, n_dec, splits, part_o, part_ml, out2,
                                 nh, nkv, d, page, window, 1 / math.sqrt(d), pos, slots, inv, write)
            assert torch.equal(out1, out2), (splits, write)
            bits = lambda c: c.view(torch.int16)                          # NaN rows compare as bits
            assert torch.equal(bits(k1), bits(k2)) and torch.equal(bits(v1), bits(v2)), (splits, write)
            assert torch.equal(x2, rows)                                  # the projection output is left alone
            if write:
                assert not torch.equal(bits(k1), bits(kc))


def test_attn_decode_rope_refuses_what_it_cannot_do(ops, cuda_device):
    from gollmgo_b200.csrc.ops import KernelError
    assert not ops.attn_decode_rope_ok(torch.float32, 8, 2, 128, torch.ones(64, dtype=torch.float64), False)
    assert not ops.attn_decode_rope_ok(torch.bfloat16, 8, 2, 80, torch.ones(40, dtype=torch.float64), False)
    assert not ops.attn_decode_rope_ok(torch.bfloat16, 34, 2, 128, torch.ones(64, dtype=torch.float64), False)
    assert not ops.attn_decode_rope_ok(torch.bfloat16, 8, 2, 128, torch.ones(32, dtype=torch.float64), False)
    assert not ops.attn_decode_rope_ok(torch.bfloat16, 8, 2, 128, torch.ones(64, dtype=torch.float64), True)
    assert ops.attn_decode_rope_ok(torch.bfloat16, 8, 2, 128, torch.ones(64, dtype=torch.float64), False)
    x = torch.zeros(1, 12 * 80, device="cuda", dtype=torch.bfloat16)
    c = torch.zeros(2, 2, 16, 80, device="cuda", dtype=torch.bfloat16)
    i = torch.zeros(4, dtype=torch.int32, device="cuda")
    with pytest.raises(KernelError):
        ops.attn_decode_rope(x, c, c, i, 1, i, i, i, 1, 1, torch.empty(4000, device="cuda"),
                             torch.empty(100, device="cuda"), torch.empty(1, 8 * 80, device="cuda", dtype=torch.bfloat16),
                             8, 2, 80, 16, 0, 0.1, i, i, torch.ones(40, dtype=torch.float64, device="cuda"))


@pytest.mark.parametrize("allow_mma", [False, True, "tc", "tc1", "tc2"])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d,page,window", [
    (4, 2, 16, 16, 0), (4, 1, 32, 8, 0), (5, 5, 48, 32, 24), (32, 8, 128, 16, 0), (6, 3, 96, 16, 40),
    (6, 2, 64, 8, 0), (3, 1, 64, 32, 50), (5, 5, 128, 16, 70), (2, 1, 128, 8, 0), (4, 4, 128, 64, 130),
    (8, 2, 64, 16, 0), (4, 2, 128, 64, 90), (12, 2, 64, 32, 33), (16, 4, 128, 16, 0), (20, 2, 128, 128, 300)])
def test_attn_prefill(ops, cuda_device, dtype, nh, nkv, d, page, window, allow_mma):
    """Portions of several sequences in one launch: (cached before, portion length).
    "tc": the best tcgen05 kernel for the shape (two heads of a kv head per CTA in steps of 128
    keys where the heads come in even groups); "tc2": the same in steps of 64 keys; "tc1": the
    tcgen05 kernel with one head per CTA."""
    if allow_mma is True and not (dtype == torch.bfloat16 and d in (64, 128)):
        pytest.skip("the mma.sync kernel takes bfloat16 with head size 64 or 128")
    if allow_mma in ("tc", "tc1", "tc2") and not (dtype == torch.bfloat16 and d in (64, 128)):
        pytest.skip("the tcgen05 kernels take bfloat16 with head size 64 or 128")
    if allow_mma in ("tc1", "tc2") and (nh // nkv) % 2:
        pytest.skip("odd groups of heads: \"tc\" already is the one-head kernel")
    torch.manual_seed(5)
    shapes = [(0, 1), (0, 2), (0, 16), (0, 17), (5, 2), (13, 40), (64, 64), (100, 33), (250, 3), (0, 130),
              (1, 63), (63, 65), (0, 64), (7, 200), (0, 128), (127, 129), (300, 260), (2100, 700)]
    seqs, qs, refs, q_lens = [], [], [], []
    for i, (start, n) in enumerate(shapes):
        ctx = start + n
        k, v = torch.randn(ctx, nkv, d, device="cuda"), torch.randn(ctx, nkv, d, device="cuda")
        q = torch.randn(n, nh, d, device="cuda")
        lo = max(0, ctx - window) if window else 0
        far = [lo, start, max(lo, start - 1), ctx - 1][i % 4]
        spike(q, k, v, i % nh, (i % nh) // (nh // nkv), min(far, ctx - 1))
        q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
        seqs.append((k, v)), qs.append(q), q_lens.append(n)
        refs.append(ref_attention(q.float(), k.float(), v.float(), start, window))
    kc, vc, bt, stride = paged(seqs, page, sum(-(-(s + n) // page) for s, n in shapes) + 3, nkv, d, dtype, 3)
    T = sum(q_lens)
    # q lives inside a wider row, as in the engine's qkv buffer
    width = nh * d + 32
    buf = torch.randn(T, width, device="cuda").to(dtype)
    buf[:, :nh * d] = torch.cat(qs).reshape(T, nh * d)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device="cuda")
    ctx_t = torch.tensor([s + n for s, n in shapes], dtype=torch.int32, device="cuda")
    tiles = [(b, q0) for b, n in enumerate(q_lens) for q0 in range(0, n, 16)]
    random.Random(6).shuffle(tiles)
    tile_seq = torch.tensor([t[0] for t in tiles], dtype=torch.int32, device="cuda")
    tile_q0 = torch.tensor([t[1] for t in tiles], dtype=torch.int32, device="cuda")
    tiles64 = [(b, q0) for b, n in enumerate(q_lens) for q0 in range(0, n, 64)]
    random.Random(7).shuffle(tiles64)
    t64_seq = torch.tensor([t[0] for t in tiles64], dtype=torch.int32, device="cuda")
    t64_q0 = torch.tensor([t[1] for t in tiles64], dtype=torch.int32, device="cuda")
    tiles128 = [(b, q0) for b, n in enumerate(q_lens) for q0 in range(0, n, 128)]
    random.Random(8).shuffle(tiles128)
    t128_seq = torch.tensor([t[0] for t in tiles128], dtype=torch.int32, device="cuda")
    t128_q0 = torch.tensor([t[1] for t in tiles128], dtype=torch.int32, device="cuda")
    out = torch.zeros(T, nh * d, device="cuda", dtype=dtype)
    ops.attn_prefill(buf, width, kc, vc, bt, stride, cu, ctx_t, tile_seq, tile_q0, len(tiles), out,
                     nh, nkv, d, page, window, 1 / math.sqrt(d), t64_seq, t64_q0, len(tiles64),
                     allow_mma=bool(allow_mma), tile128_seq=t128_seq, tile128_q0=t128_q0,
                     num_tiles128=len(tiles128), allow_tc={"tc": 1, "tc1": 2, "tc2": 3}.get(allow_mma, 0))
    if allow_mma in ("tc", "tc1", "tc2"):
        ops.check_tc_status("cuda")
    torch.testing.assert_close(out.double(), torch.cat(refs).reshape(T, nh * d), **tol(dtype))


def test_the_prompt_kernel_in_steps_of_128_keys_is_the_one_that_runs(ops, cuda_device):
    """It needs the register count the compiler gave the kernel to cover what its warps hand
    back and take (a build where it does not falls back to steps of 64 keys without a word):
    on this build it must be there, for the shapes of the benchmarks."""
    assert ops.attn_prefill_choice(torch.bfloat16, 128, 16, 32, 8) == 3
    assert ops.attn_prefill_choice(torch.bfloat16, 64, 16, 32, 8) == 3
    assert ops.attn_prefill_choice(torch.bfloat16, 128, 128, 4, 2) == 3
    assert ops.attn_prefill_choice(torch.bfloat16, 128, 16, 5, 5) == 1          # odd groups: one head per CTA
    assert ops.attn_prefill_choice(torch.bfloat16, 96, 16, 4, 2) == 0
    assert ops.attn_prefill_choice(torch.float32, 128, 16, 4, 2) == 0


def test_attention_refuses_what_it_cannot_do(ops, cuda_device):
    z = torch.zeros(4, device="cuda")
    zi = torch.zeros(4, dtype=torch.int32, device="cuda")
    with pytest.raises(ops.KernelError, match="head size"):
        ops.attn_prefill(z, 1, z, z, zi, 1, zi, zi, zi, zi, 1, z, 2, 1, 272, 16, 0, 1.0)
    with pytest.raises(ops.KernelError, match="multiple"):
        ops.attn_prefill(z, 1, z, z, zi, 1, zi, zi, zi, zi, 1, z, 5, 2, 16, 16, 0, 1.0)


# ---------------------------------------------------------------- sampling
def test_argmax_first_maximum_wins(ops, cuda_device):
    V = 128256 + 3
    logits = torch.randn(5, V, device="cuda")
    logits[0, 77] = logits[0, 90000] = 50.0
    logits[1, V - 1] = 60.0
    logits[2, 0] = 60.0
    logits[3] = -1.0
    out = torch.empty(5, dtype=torch.int32, device="cuda")
    ops.argmax(logits, out)
    assert out.tolist() == [77, V - 1, 0, 0, int(logits[4].argmax())]


@pytest.mark.parametrize("V", [1013, 16385, 50257, 128256])
def test_sample_matches_the_plain_sampler(ops, cuda_device, V):
    """(From 16384 entries a row is spread over a cluster of CTAs: another kernel.)"""
    import plain_llama as P
    torch.manual_seed(7)
    R = 24
    logits = (torch.randn(R, V) * 2.5).cuda()
    temps = [0.0, 0.8, 1.0, 1.3, 0.5, 2.0] * 4
    top_k = [0, 0, 50, 0, 7, 1] * 4
    top_p = [0.0, 0.0, 0.0, 0.9, 0.7, 0.0] * 4
    seeds = list(range(100, 100 + R))
    draws = [i % 5 for i in range(R)]
    out = torch.empty(R, dtype=torch.int32, device="cuda")
    dev = lambda x, dt: torch.tensor(x, dtype=dt, device="cuda")
    ops.sample(logits, dev(temps, torch.float32), dev(top_k, torch.int32), dev(top_p, torch.float32),
               dev(seeds, torch.int64), dev(draws, torch.int64), out)
    host = logits.cpu()
    agree = 0
    for r in range(R):
        want = P.sample(host[r], temps[r], seeds[r], draws[r], top_k[r], top_p[r])
        got = int(out[r])
        if got == want:
            agree += 1
            continue
        # a draw that falls within rounding of a boundary may land on the neighbour
        p = P.probabilities(host[r], temps[r], top_k[r], top_p[r])
        u = P.uniform_draw(seeds[r], draws[r])
        cum = torch.cumsum(p, 0)
        assert p[got] > 0 and abs(float(cum[got]) - u) < 1e-4 or abs(float(cum[got] - p[got]) - u) < 1e-4, \
            f"row {r}: kernel chose {got}, plain {want}"
    assert agree >= R - 2
    again = torch.empty_like(out)
    ops.sample(logits, dev(temps, torch.float32), dev(top_k, torch.int32), dev(top_p, torch.float32),
               dev(seeds, torch.int64), dev(draws, torch.int64), again)
    assert torch.equal(out, again)


@pytest.mark.parametrize("V", [50, 20000])
def test_sample_statistics_and_seeds(ops, cuda_device, V):
    R = 4000
    row = torch.linspace(-2, 2, V) if V == 50 else torch.cat([torch.linspace(-2, 2, 50), torch.full((V - 50,), -60.0)])
    logits = row.repeat(R, 1).cuda()
    dev = lambda x, dt: torch.tensor(x, dtype=dt, device="cuda")
    out = torch.empty(R, dtype=torch.int32, device="cuda")
    args = (dev([0.7] * R, torch.float32), None, None)
    ops.sample(logits, *args, dev([5] * R, torch.int64), dev(list(range(R)), torch.int64), out)
    freq = torch.bincount(out.long().cpu(), minlength=V).double() / R
    p = torch.softmax(row.double() / 0.7, 0)
    assert float((freq - p).abs().max()) < 0.025
    again = torch.empty_like(out)
    ops.sample(logits, *args, dev([5] * R, torch.int64), dev(list(range(R)), torch.int64), again)
    assert torch.equal(out, again)                                     # same seed and draw: same token
    other = torch.empty_like(out)
    ops.sample(logits, *args, dev([6] * R, torch.int64), dev(list(range(R)), torch.int64), other)
    assert not torch.equal(out, other)


# ---------------------------------------------------------------- products for a few tokens
@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(48, 64), (100, 120), (4096, 4096), (1000, 14336 + 8)])
def test_gemm_small_m(ops, cuda_device, M, N, K):
    g = torch.Generator(device="cuda").manual_seed(M * 1000 + N)
    x_wide = (torch.randn(M, K + 16, device="cuda", generator=g)).to(torch.bfloat16)
    x = x_wide[:, :K]                                                   # rows with a stride wider than K
    w = (torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)).to(torch.bfloat16)
    ref = x.float() @ w.float().T
    out32 = torch.empty(M, N, device="cuda")
    ops.gemm_small_m(x, w, out32)
    torch.testing.assert_close(out32, ref, rtol=1e-4, atol=1e-4)       # float32 accumulate of bf16 inputs
    out16 = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    ops.gemm_small_m(x, w, out16)
    assert torch.equal(out16, out32.to(torch.bfloat16))
    # a spike in one far column of K must arrive in exactly one output
    x2, w2 = x.clone(), w.clone()
    x2[M - 1, K - 3] = 64.0
    w2[N - 1, K - 3] = 8.0
    ops.gemm_small_m(x2, w2, out32)
    torch.testing.assert_close(out32, x2.float() @ w2.float().T, rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize("M", [1, 8, 13])
@pytest.mark.parametrize("I,K", [(44, 64), (352, 128), (14336, 4096)])
def test_gemm_small_m_gated(ops, cuda_device, M, I, K):
    g = torch.Generator(device="cuda").manual_seed(M + I)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * I, K, device="cuda", generator=g) * (2.0 / math.sqrt(K))).to(torch.bfloat16)
    out = torch.empty(M, I, device="cuda", dtype=torch.bfloat16)
    ops.gemm_small_m(x, w, out, gated=True)
    gu = x.float() @ w.float().T
    gate, up = gu[:, :I], gu[:, I:]
    ref = gate / (1 + torch.exp(-gate)) * up
    torch.testing.assert_close(out.float(), ref.to(torch.bfloat16).float(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("M", [1, 8, 11])
@pytest.mark.parametrize("H,I", [(48, 104), (4096, 1024), (1000, 264)])
def test_gemm_small_m_with_norms_folded_in(ops, cuda_device, M, H, I):
    """A product that adds to the residual and prepares the next norm, then a (gated) product
    that takes the unnormalised input: together the same as add, RMSNorm, product."""
    g = torch.Generator(device="cuda").manual_seed(M + H)
    eps = 3e-6
    a = torch.randn(M, I, device="cuda", generator=g).to(torch.bfloat16)
    w_down = (torch.randn(H, I, device="cuda", generator=g) / math.sqrt(I)).to(torch.bfloat16)
    resid0 = torch.randn(M, H, device="cuda", generator=g) * 3
    norm_w = 1 + 0.2 * torch.randn(H, device="cuda", generator=g)
    w_gu = (torch.randn(2 * I, H, device="cuda", generator=g) * (2.0 / math.sqrt(H))).to(torch.bfloat16)
    w_q = (torch.randn(I, H, device="cuda", generator=g) / math.sqrt(H)).to(torch.bfloat16)
    # reference in float64
    h = resid0.double() + a.double() @ w_down.double().T
    xn = h * torch.rsqrt((h * h).mean(-1, keepdim=True) + eps) * norm_w.double()
    gu = xn @ w_gu.double().T
    ref_gated = gu[:, :I] / (1 + torch.exp(-gu[:, :I])) * gu[:, I:]
    ref_q = xn @ w_q.double().T
    # the kernels
    resid = resid0.clone()
    scaled = torch.empty(M, H, device="cuda", dtype=torch.bfloat16)
    partials = torch.full((-(-H // 16), 16), float("nan"), device="cuda")
    ops.gemm_small_m(a, w_down, scaled, resid=resid, norm_w=norm_w, out_partials=partials)
    torch.testing.assert_close(resid.double(), h, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(scaled.double(), (h * norm_w.double()), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(partials[:, :M].sum(0).double(), (h * h).sum(-1), rtol=1e-5, atol=1e-5)
    out_g = torch.empty(M, I, device="cuda", dtype=torch.bfloat16)
    ops.gemm_small_m(scaled, w_gu, out_g, gated=True, in_partials=partials, hidden=H, eps=eps)
    out_q = torch.empty(M, I, device="cuda", dtype=torch.bfloat16)
    ops.gemm_small_m(scaled, w_q, out_q, in_partials=partials, hidden=H, eps=eps)
    out_f = torch.empty(M, I, device="cuda", dtype=torch.float32)
    ops.gemm_small_m(scaled, w_q, out_f, in_partials=partials, hidden=H, eps=eps)
    scale = ref_q.abs().max().item()
    assert (out_q.double() - ref_q).abs().max().item() <= 2e-2 * scale
    assert (out_f.double() - ref_q).abs().max().item() <= 1e-2 * scale        # only x is rounded to bfloat16
    assert (out_g.double() - ref_gated).abs().max().item() <= 2e-2 * ref_gated.abs().max().item()
    # twice the same: no atomics anywhere
    resid2, scaled2, partials2 = resid0.clone(), torch.empty_like(scaled), torch.empty_like(partials)
    ops.gemm_small_m(a, w_down, scaled2, resid=resid2, norm_w=norm_w, out_partials=partials2)
    assert torch.equal(resid, resid2) and torch.equal(scaled, scaled2) and torch.equal(partials[:, :M], partials2[:, :M])


@pytest.mark.parametrize("M", [1, 17, 32, 33, 50, 64])
@pytest.mark.parametrize("N,K", [(48, 64), (100, 120), (4096, 4096), (1000, 14336 + 8), (6144, 4096), (130, 72),
                                 (28672, 512), (37991, 200), (9475, 64), (20000, 1024)])
def test_gemm_mid_m(ops, cuda_device, M, N, K):
    """Few rows of w (slabs of 128 rows, K split over a cluster) and many (one CTA per SM, slabs
    of whatever height fills the machine, one or two boxes; several rounds; an odd N, where
    outputs are stored one by one)."""
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)).to(torch.bfloat16)
    ref = x.double() @ w.double().T
    for dt in (torch.bfloat16, torch.float32):
        out = torch.full((M, N), float("nan"), device="cuda", dtype=dt)
        ops.gemm_mid_m(x, w, out)
        ops.check_tc_status("cuda")
        t = dict(rtol=1e-2, atol=1e-2) if dt == torch.bfloat16 else dict(rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(out.double(), ref, **t)
    # x as rows of a wider buffer, as the engine's workspaces are
    wide = torch.randn(M, K + 64, device="cuda", generator=g).to(torch.bfloat16)
    out = torch.empty(M, N, device="cuda", dtype=torch.float32)
    ops.gemm_mid_m(wide[:, :K], w, out)
    torch.testing.assert_close(out.double(), wide[:, :K].double() @ w.double().T, rtol=1e-4, atol=1e-4)
    ops.check_tc_status("cuda")


@pytest.mark.parametrize("M", [17, 40, 64])
@pytest.mark.parametrize("I,K", [(44, 64), (352, 128), (14336, 4096), (200, 72), (19001, 136), (8192, 2048)])
def test_gemm_mid_m_gated(ops, cuda_device, M, I, K):
    g = torch.Generator(device="cuda").manual_seed(M + I)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * I, K, device="cuda", generator=g) * (2.0 / math.sqrt(K))).to(torch.bfloat16)
    out = torch.full((M, I), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.gemm_mid_m(x, w, out, gated=True)
    ops.check_tc_status("cuda")
    gu = x.float() @ w.float().T
    gate, up = gu[:, :I], gu[:, I:]
    ref = gate / (1 + torch.exp(-gate)) * up
    torch.testing.assert_close(out.float(), ref.to(torch.bfloat16).float(), rtol=1e-2, atol=1e-2)


def test_gemm_small_m_refuses_what_it_cannot_do(ops, cuda_device):
    x = torch.zeros(17, 64, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(32, 64, device="cuda", dtype=torch.bfloat16)
    assert not ops.small_m_ok(x, w)
    with pytest.raises(ops.KernelError, match="at most 16"):
        ops.gemm_small_m(x, w, torch.empty(17, 32, device="cuda", dtype=torch.bfloat16))
    assert not ops.small_m_ok(x[:4, :60], w[:, :60].contiguous())       # K not a multiple of 8


# ---------------------------------------------------------------- products on tcgen05
@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 256), (256, 512, 4096), (200, 300, 136),
                                   (2048, 6144, 4096), (77, 4096, 14336), (1, 256, 64)])
def test_gemm_tc(ops, cuda_device, M, N, K, pair):
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    x_wide = torch.randn(M, K + 24, device="cuda", generator=g).to(torch.bfloat16)
    x = x_wide[:, :K]
    w = (torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)).to(torch.bfloat16)
    ref = x.float() @ w.float().T
    out32 = torch.full((M, N), float("nan"), device="cuda")
    ops.gemm_tc(x, w, out32, pair=pair)
    ops.check_tc_status("cuda")
    torch.testing.assert_close(out32, ref, rtol=2e-4, atol=2e-4)
    out16 = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    ops.gemm_tc(x, w, out16, pair=pair)
    ops.check_tc_status("cuda")
    assert torch.equal(out16, out32.to(torch.bfloat16))
    # one large entry in a far corner of K must reach exactly one output
    x2, w2 = x.clone(), w.clone()
    x2[M - 1, K - 5] = 64.0
    w2[N - 1, K - 5] = 8.0
    ops.gemm_tc(x2, w2, out32, pair=pair)
    torch.testing.assert_close(out32, x2.float() @ w2.float().T, rtol=2e-4, atol=2e-3)


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("M,I,K", [(128, 128, 64), (300, 352, 128), (2048, 14336, 4096), (65, 200, 72)])
def test_gemm_tc_gated(ops, cuda_device, M, I, K, pair):
    g = torch.Generator(device="cuda").manual_seed(M + I)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * I, K, device="cuda", generator=g) * (2.0 / math.sqrt(K))).to(torch.bfloat16)
    out = torch.full((M, I), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.gemm_tc(x, w, out, gated=True, pair=pair)
    ops.check_tc_status("cuda")
    gu = x.float() @ w.float().T
    gate, up = gu[:, :I], gu[:, I:]
    ref = gate / (1 + torch.exp(-gate)) * up
    torch.testing.assert_close(out.float(), ref.to(torch.bfloat16).float(), rtol=1e-2, atol=1e-2)


def test_gemm_tc_bounded_waits_report_and_return(ops, cuda_device):
    """No barrier inside the tcgen05 kernels is waited on without a limit.  With the loads
    withheld nothing a consumer waits for ever arrives: the kernel must give up, say so in its
    status word, free its tensor memory and return, and the next launch must work as usual."""
    import time
    x = torch.randn(128, 256, device="cuda").to(torch.bfloat16)
    w = torch.randn(256, 256, device="cuda").to(torch.bfloat16)
    out = torch.zeros(128, 256, device="cuda", dtype=torch.bfloat16)
    torch.cuda.synchronize()
    t0 = time.time()
    ops.gemm_tc_withheld(x, w, out)
    torch.cuda.synchronize()
    assert time.time() - t0 < 30
    with pytest.raises(ops.KernelError, match="gave up waiting"):
        ops.check_tc_status("cuda")
    ops.check_tc_status("cuda")                                        # the word was cleared
    ops.gemm_tc(x, w, out)                                             # tensor memory was given back
    ops.check_tc_status("cuda")
    torch.testing.assert_close(out.float(), (x.float() @ w.float().T).to(torch.bfloat16).float(), rtol=1e-2, atol=1e-2)
