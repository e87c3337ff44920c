"""The entry point for callers that cannot allocate device memory
(gg_attn_decode_noalloc, csrc/no_alloc.h): called through its exported C symbol,
twice in a row, and compared with the ordinary entry point that takes scratch
buffers from the caller and with a plain float64 attention.  The second call uses other
inputs, so anything the first call left in the built-in scratch would show.  One case has
more slices than a thread-block cluster holds: only then does the bfloat16 kernel put its
partial results into the built-in array (up to eight slices merge inside a cluster, through
shared memory).  This file sorts last on purpose: if it fails, every other test has already
run."""
import ctypes
import math
import random

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_PART_O = 1 << 20


def _case(seed, nh, nkv, d, page, ctxs, dtype):
    g = torch.Generator(device="cuda").manual_seed(seed)
    B = len(ctxs)
    pages = sum(-(-c // page) for c in ctxs) + 2
    order = list(range(pages))
    random.Random(seed).shuffle(order)
    kc = torch.randn(pages, nkv, page, d, device="cuda", generator=g).to(dtype)
    vc = torch.randn(pages, nkv, page, d, device="cuda", generator=g).to(dtype)
    stride = max(-(-c // page) for c in ctxs)
    bt = torch.full((B, stride), -1, dtype=torch.int32)
    for b, c in enumerate(ctxs):
        for lp in range(-(-c // page)):
            bt[b, lp] = order.pop()
    q = torch.randn(B, nh * d, device="cuda", generator=g).to(dtype)
    return dict(q=q, kc=kc, vc=vc, bt=bt.cuda(), stride=stride,
                cu=torch.arange(B + 1, dtype=torch.int32, device="cuda"),
                ctx=torch.tensor(ctxs, dtype=torch.int32, device="cuda"),
                dec=torch.arange(B, dtype=torch.int32, device="cuda"), B=B)


def _plain_attention(c, nh, nkv, d, page):
    """softmax(q k^T / sqrt(d)) v over each sequence's pages, in float64."""
    out = torch.empty(c["B"], nh * d, dtype=torch.float64, device="cuda")
    group = nh // nkv
    for b in range(c["B"]):
        n = int(c["ctx"][b])
        pages = c["bt"][b, :-(-n // page)].long()
        k = c["kc"][pages].double().permute(1, 0, 2, 3).reshape(nkv, -1, d)[:, :n]      # [nkv, n, d]
        v = c["vc"][pages].double().permute(1, 0, 2, 3).reshape(nkv, -1, d)[:, :n]
        q = c["q"][b].double().view(nkv, group, d)
        p = torch.softmax(q @ k.transpose(1, 2) / math.sqrt(d), dim=-1)
        out[b] = (p @ v).reshape(-1)
    return out


@pytest.mark.parametrize("dtype,nh,nkv,d,page,splits", [
    (torch.bfloat16, 32, 8, 128, 16, 4),      # tensor-core kernel, slices merged inside a cluster
    (torch.bfloat16, 32, 8, 128, 16, 11),     # more slices than a cluster holds: partial results in the built-in array
    (torch.float32, 6, 2, 48, 8, 3),          # general kernel
])
def test_no_alloc_entry_matches_the_ordinary_one(cuda_device, dtype, nh, nkv, d, page, splits):
    from gollmgo_b200.csrc import ops
    lib = ctypes.CDLL(ops.library_file())             # the exported C symbols, nothing else
    lib.gg_last_error.restype = ctypes.c_char_p
    code = ops.dtype_code(dtype)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    tol = dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    for seed, ctxs in ((1, [300, 17, 64, 129, 1]), (2, [5, 700, 333, 64, 90])):      # two calls in a row
        c = _case(seed, nh, nkv, d, page, ctxs, dtype)
        common = lambda: (p(c["q"]), ctypes.c_longlong(nh * d), p(c["kc"]), p(c["vc"]), code, p(c["bt"]),
                          c["stride"], p(c["cu"]), p(c["ctx"]), p(c["dec"]), c["B"], splits)
        tail = (nh, nkv, d, page, 0, ctypes.c_float(1 / math.sqrt(d)), 1, stream)
        want = torch.zeros(c["B"], nh * d, device="cuda", dtype=dtype)
        part_o = torch.empty(c["B"] * nh * splits * d, device="cuda")
        part_ml = torch.empty(c["B"] * nh * splits * 2, device="cuda")
        rc = lib.gg_attn_decode(*common(), p(part_o), p(part_ml), p(want), *tail)
        assert rc == 0, lib.gg_last_error().decode()
        got = torch.zeros_like(want)
        before = torch.cuda.memory_allocated()
        rc = lib.gg_attn_decode_noalloc(*common(), p(got), *tail)
        assert rc == 0, lib.gg_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.isfinite(got.float()).all()
        torch.testing.assert_close(got.float(), want.float(), **tol)
        torch.testing.assert_close(got.double(), _plain_attention(c, nh, nkv, d, page), **tol)


def test_no_alloc_entry_refuses_what_does_not_fit(cuda_device):
    from gollmgo_b200.csrc import ops
    lib = ctypes.CDLL(ops.library_file())
    lib.gg_last_error.restype = ctypes.c_char_p
    z = ctypes.c_void_p(0)
    n_dec, nh, d, splits = 64, 32, 128, 8             # 2,097,152 floats of partial outputs: too many
    assert n_dec * nh * splits * d > MAX_PART_O
    rc = lib.gg_attn_decode_noalloc(z, ctypes.c_longlong(nh * d), z, z, 1, z, 1, z, z, z, n_dec, splits, z,
                                    nh, 8, d, 16, 0, ctypes.c_float(0.1), 1, z)
    assert rc != 0 and "exceed the built-in scratch" in lib.gg_last_error().decode()
