"""Python face of the CUDA library: one function per launcher, taking torch tensors.

There is no CPU fallback and no other implementation behind these names: if the
library cannot be built or loaded, importing a function's first use raises.  All
launches go to torch's current CUDA stream, so they can be captured in a graph.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    """A launcher refused its arguments or CUDA reported an error."""


_LIB = None


def lib():
    global _LIB
    if _LIB is None:
        path = build.ensure_built()
        try:
            handle = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load the CUDA library {path}: {e}") from None
        handle.gg_last_error.restype = ctypes.c_char_p
        _LIB = handle
    return _LIB


def library_file() -> str:
    lib()
    return build.library_path()


def _p(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current CUDA stream of the current device as a pointer (asked on every launch: a graph
    capture runs on a stream of its own).  The raw accessor costs a tenth of building a
    torch.cuda.Stream object, which matters at a few hundred launches per prompt step."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


launches = 0          # kernels of this library launched by this process (a captured graph counts once)


def _check(rc: int, n: int = 1) -> None:
    global launches
    if rc != 0:
        raise KernelError(lib().gg_last_error().decode())
    launches += n


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dt}")


def _cuda(*tensors):
    for t in tensors:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise KernelError("kernel arguments must be contiguous CUDA tensors")


def device_capability() -> int:
    return int(lib().gg_device_capability())


def embed_gather(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor,
                 bad_id: Optional[torch.Tensor] = None, token_src: Optional[torch.Tensor] = None,
                 prev_tokens: Optional[torch.Tensor] = None) -> None:
    """out[t, :] = float32(table[id_t, :]); ids int32 [T], out float32 [T, H].  Where
    token_src[t] >= 0 the id is prev_tokens[token_src[t]] (a token still on the device)."""
    _cuda(ids, table, out, token_src, prev_tokens)
    T, (V, H) = ids.numel(), table.shape
    if out.dtype != torch.float32 or out.shape[-1] != H or ids.dtype != torch.int32:
        raise KernelError("embed_gather: out must be float32 [T, H], ids int32")
    _check(lib().gg_embed_gather(_p(ids), _p(table), dtype_code(table.dtype), _p(out),
                                 T, H, V, _p(bad_id), _p(token_src), _p(prev_tokens), _stream()))


def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                out: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None,
                write_back: bool = True) -> None:
    """x = resid[r] (+ delta[r]); resid[r] = x if write_back; out[i] = rmsnorm(x) * weight,
    r = rows[i] if rows is given else i.  resid float32, weight float32, out/delta same dtype.
    ``rows`` and ``weight`` are read before the kernel ahead of this one has finished: they must
    not be that kernel's output (the engine gives the step's packed row list)."""
    _cuda(resid, delta, weight, out, rows)
    H = resid.shape[-1]
    n = rows.numel() if rows is not None else out.shape[0]
    if resid.dtype != torch.float32 or weight.dtype != torch.float32 or weight.numel() != H:
        raise KernelError("add_rmsnorm: residual and weight must be float32 of one width")
    if delta is not None and delta.dtype != out.dtype:
        raise KernelError("add_rmsnorm: delta and out differ in dtype")
    _check(lib().gg_add_rmsnorm(_p(resid), _p(delta), _p(weight), _p(out), dtype_code(out.dtype),
                                _p(rows), n, H, ctypes.c_float(eps), int(write_back), _stream()))


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    _cuda(gate_up, out)
    T, I = out.shape
    if gate_up.shape != (T, 2 * I) or gate_up.dtype != out.dtype:
        raise KernelError("silu_mul: input must be [T, 2I] of the output's dtype")
    _check(lib().gg_silu_mul(_p(gate_up), _p(out), dtype_code(out.dtype), T, I, _stream()))


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, slot_mapping: Optional[torch.Tensor],
                  inv_freq: Optional[torch.Tensor], kcache: Optional[torch.Tensor],
                  vcache: Optional[torch.Tensor], nh: int, nkv: int, d: int, page_size: int,
                  interleaved: bool = False, write_cache: bool = True) -> None:
    """Rotate q and k heads of qkv [T, (nh+2nkv)*d] in place and scatter k, v into the
    paged cache [pages, nkv, page_size, d] at slot_mapping[t].  ``positions``, ``slot_mapping``
    and ``inv_freq`` are read before the kernel ahead of this one has finished: they must not be
    that kernel's output (the engine gives the step's packed lists)."""
    _cuda(qkv, positions, slot_mapping, inv_freq, kcache, vcache)
    T = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * d:
        raise KernelError("rope_kv_write: qkv width is not (nh + 2 nkv) * d")
    if inv_freq is not None and inv_freq.dtype != torch.float64:
        raise KernelError("rope_kv_write: inverse frequencies must be float64")
    if kcache is not None and kcache.dtype != qkv.dtype:
        raise KernelError("rope_kv_write: cache and activations differ in dtype")
    rot = 2 * inv_freq.numel() if inv_freq is not None else 0
    _check(lib().gg_rope_kv_write(_p(qkv), dtype_code(qkv.dtype), _p(positions), _p(slot_mapping),
                                  _p(inv_freq), _p(kcache), _p(vcache), T, nh, nkv, d, rot,
                                  page_size, int(interleaved), int(write_cache), _stream()))


def attn_prefill(q: torch.Tensor, q_stride: int, kcache: torch.Tensor, vcache: torch.Tensor,
                 block_tables: torch.Tensor, bt_stride: int, cu_q_lens: torch.Tensor,
                 context_lens: torch.Tensor, tile_seq: torch.Tensor, tile_q0: torch.Tensor,
                 num_tiles: int, out: torch.Tensor, nh: int, nkv: int, d: int, page_size: int,
                 window: int, scale: float, tile64_seq: Optional[torch.Tensor] = None,
                 tile64_q0: Optional[torch.Tensor] = None, num_tiles64: int = 0,
                 allow_mma: bool = True, tile128_seq: Optional[torch.Tensor] = None,
                 tile128_q0: Optional[torch.Tensor] = None, num_tiles128: int = 0,
                 allow_tc: bool = True) -> None:
    """Causal attention of prompt portions over the paged cache.  ``tile_*`` list tiles
    of 16 queries (general kernel), ``tile64_*`` of 64 (mma.sync kernel: bfloat16, head
    size 64 or 128), ``tile128_*`` of 128 (tcgen05 kernel: bfloat16, head size 64 or 128); the
    most specialised kernel whose list is given and that is allowed runs.  ``allow_tc``: 2 =
    only the tcgen05 kernel with one head per CTA, not the one with two heads of a kv head."""
    global tc_launched
    use_tc = allow_tc and tile128_seq is not None and kcache.dtype == torch.bfloat16 and d in (64, 128)
    if use_tc:
        tc_launched = True
    _check(lib().gg_attn_prefill(_p(q), ctypes.c_longlong(q_stride), _p(kcache), _p(vcache),
                                 dtype_code(kcache.dtype), _p(block_tables), bt_stride,
                                 _p(cu_q_lens), _p(context_lens), _p(tile_seq), _p(tile_q0),
                                 num_tiles, _p(tile64_seq), _p(tile64_q0), num_tiles64,
                                 _p(tile128_seq), _p(tile128_q0), num_tiles128, _p(out),
                                 q.shape[0], kcache.shape[0], nh, nkv, d, page_size, window,
                                 ctypes.c_float(scale), int(allow_mma), int(allow_tc),
                                 _p(tc_status(q.device)) if use_tc else ctypes.c_void_p(0), _stream()))


def attn_decode(q: torch.Tensor, q_stride: int, kcache: torch.Tensor, vcache: torch.Tensor,
                block_tables: torch.Tensor, bt_stride: int, cu_q_lens: torch.Tensor,
                context_lens: torch.Tensor, dec_seqs: torch.Tensor, n_dec: int, num_splits: int,
                part_o: torch.Tensor, part_ml: torch.Tensor, out: torch.Tensor, nh: int, nkv: int,
                d: int, page_size: int, window: int, scale: float, allow_mma: bool = True) -> None:
    """Attention of single decoded tokens, split over the context and merged."""
    if part_o.numel() < n_dec * nh * num_splits * d or part_ml.numel() < n_dec * nh * num_splits * 2:
        raise KernelError("attn_decode: scratch too small")
    _check(lib().gg_attn_decode(_p(q), ctypes.c_longlong(q_stride), _p(kcache), _p(vcache),
                                dtype_code(kcache.dtype), _p(block_tables), bt_stride,
                                _p(cu_q_lens), _p(context_lens), _p(dec_seqs), n_dec, num_splits,
                                _p(part_o), _p(part_ml), _p(out), nh, nkv, d, page_size, window,
                                ctypes.c_float(scale), int(allow_mma), _stream()), 2)


def attn_decode_rope_ok(dtype: torch.dtype, nh: int, nkv: int, d: int, inv_freq: Optional[torch.Tensor],
                        interleaved: bool) -> bool:
    """Whether attn_decode_rope takes this shape: bfloat16, head size 64 or 128, at most 16
    heads per kv head, half-split rotation over the whole head."""
    return (dtype == torch.bfloat16 and d in (64, 128) and nh // nkv <= 16 and inv_freq is not None
            and inv_freq.dtype == torch.float64 and 2 * inv_freq.numel() == d and not interleaved)


def attn_decode_rope(qkv: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                     block_tables: torch.Tensor, bt_stride: int, cu_q_lens: torch.Tensor,
                     context_lens: torch.Tensor, dec_seqs: torch.Tensor, n_dec: int, num_splits: int,
                     part_o: torch.Tensor, part_ml: torch.Tensor, out: torch.Tensor, nh: int, nkv: int,
                     d: int, page_size: int, window: int, scale: float, positions: torch.Tensor,
                     slot_mapping: Optional[torch.Tensor], inv_freq: torch.Tensor,
                     write_cache: bool = True) -> None:
    """rope_kv_write and attn_decode of single decoded tokens in one kernel: qkv is the raw
    projection output and stays as it is; k (rotated) and v land in the cache."""
    _cuda(qkv, positions, slot_mapping, inv_freq, kcache, vcache)
    if not attn_decode_rope_ok(qkv.dtype, nh, nkv, d, inv_freq, False) or kcache.dtype != qkv.dtype:
        raise KernelError("attn_decode_rope: shape or dtype not taken (see attn_decode_rope_ok)")
    if qkv.shape[1] != (nh + 2 * nkv) * d or qkv.stride(0) != qkv.shape[1]:
        raise KernelError("attn_decode_rope: qkv must be contiguous [T, (nh + 2 nkv) * d]")
    if part_o.numel() < n_dec * nh * num_splits * d or part_ml.numel() < n_dec * nh * num_splits * 2:
        raise KernelError("attn_decode_rope: scratch too small")
    if write_cache and slot_mapping is None:
        raise KernelError("attn_decode_rope: cache write without slots")
    _check(lib().gg_attn_decode_rope(_p(qkv), ctypes.c_longlong(qkv.shape[1]), _p(kcache), _p(vcache),
                                     dtype_code(kcache.dtype), _p(block_tables), bt_stride,
                                     _p(cu_q_lens), _p(context_lens), _p(dec_seqs), n_dec, num_splits,
                                     _p(part_o), _p(part_ml), _p(out), nh, nkv, d, page_size, window,
                                     ctypes.c_float(scale), _p(positions), _p(slot_mapping), _p(inv_freq),
                                     int(write_cache), _stream()), 2)


ATTN_FLAT_MAX_SEQS = 1024   # decoded tokens attn_decode_flat takes in one launch (FLAT_MAX_SEQS in attention_mma.cu)


def attn_prefill_choice(dtype: torch.dtype, d: int, page_size: int, nh: int, nkv: int) -> int:
    """Which tcgen05 prompt kernel attn_prefill(allow_tc=True) runs for a shape on this build and
    device: 3 = two heads per CTA in steps of 128 keys, 2 = the same in steps of 64, 1 = one head
    per CTA, 0 = none."""
    return int(lib().gg_attn_prefill_choice(dtype_code(dtype), d, page_size, nh, nkv))


def attn_decode_flat_ctas(d: int) -> int:
    """CTAs that attn_decode_flat launches for head size d (for sizing its scratch)."""
    return int(lib().gg_attn_decode_flat_ctas(d))


def attn_decode_flat_pieces(n_dec: int, nh: int, nkv: int, d: int) -> int:
    """Partial results attn_decode_flat may leave: scratch part_o holds pieces * 16 * d floats,
    part_ml pieces * 16 * 2."""
    return n_dec * nkv * -(-(nh // nkv) // 16) + attn_decode_flat_ctas(d)


def attn_decode_flat_prefix_ints(n_dec: int, nh: int, nkv: int) -> int:
    """int32 scratch of attn_decode_flat: the tiles before each token, then for each (kv head
    chunk, token) pair the CTAs that hold its first and last piece."""
    return n_dec + 1 + 2 * n_dec * nkv * -(-(nh // nkv) // 16)


def attn_decode_flat(q: torch.Tensor, q_stride: int, kcache: torch.Tensor, vcache: torch.Tensor,
                     block_tables: torch.Tensor, bt_stride: int, cu_q_lens: torch.Tensor,
                     context_lens: torch.Tensor, dec_seqs: torch.Tensor, n_dec: int,
                     part_o: torch.Tensor, part_ml: torch.Tensor, prefix: torch.Tensor, out: torch.Tensor,
                     nh: int, nkv: int, d: int, page_size: int, window: int, scale: float) -> None:
    """Attention of single decoded tokens for large batches (bfloat16, head size 64 or 128):
    the 64-key tiles of all (token, kv head) pairs are cut into equal ranges, one per CTA,
    and merged by a second kernel.  ``prefix``: int32 scratch of attn_decode_flat_prefix_ints()."""
    pieces = attn_decode_flat_pieces(n_dec, nh, nkv, d)
    if part_o.numel() < pieces * 16 * d or part_ml.numel() < pieces * 16 * 2 \
            or prefix.numel() < attn_decode_flat_prefix_ints(n_dec, nh, nkv):
        raise KernelError("attn_decode_flat: scratch too small")
    if prefix.dtype != torch.int32 or part_o.dtype != torch.float32 or part_ml.dtype != torch.float32:
        raise KernelError("attn_decode_flat: scratch of the wrong type")
    _check(lib().gg_attn_decode_flat(_p(q), ctypes.c_longlong(q_stride), _p(kcache), _p(vcache),
                                     dtype_code(kcache.dtype), _p(block_tables), bt_stride,
                                     _p(cu_q_lens), _p(context_lens), _p(dec_seqs), n_dec,
                                     _p(part_o), _p(part_ml), _p(prefix), prefix.numel(), _p(out), nh, nkv, d, page_size,
                                     window, ctypes.c_float(scale), _stream()), 2)


ATTN_MAX_CLUSTER = 8  # largest count of slices that the decode kernel merges inside a cluster


def attn_decode_cluster_capacity(dtype: torch.dtype, d: int, splits: int, group: int) -> int:
    """Clusters of `splits` decode CTAs the device holds at once, with `group` query heads
    to a kv head; 0 where attn_decode merges with a kernel of its own instead."""
    if dtype not in (torch.bfloat16, torch.float32):
        return 0
    return int(lib().gg_attn_decode_cluster_capacity(dtype_code(dtype), d, splits, group))


SMALL_M = 16          # most tokens gemm_small_m takes


def small_m_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether out = x @ w^T can go through gemm_small_m."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_cuda
            and 0 < x.shape[0] <= SMALL_M and x.shape[1] % 8 == 0 and x.stride(1) == 1
            and x.stride(0) % 8 == 0 and w.is_contiguous())


def gemm_small_m(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gated: bool = False,
                 in_partials: Optional[torch.Tensor] = None, hidden: int = 0, eps: float = 0.0,
                 resid: Optional[torch.Tensor] = None, norm_w: Optional[torch.Tensor] = None,
                 out_partials: Optional[torch.Tensor] = None) -> None:
    """out[M, N] = x[M, K] @ w[N, K]^T for M <= 16 (bfloat16 in, float32 accumulate); out is
    bfloat16 or float32.  ``gated``: w is [2N, K] (gate rows, then up rows) and
    out = silu(x Wg^T) * (x Wu^T) in bfloat16.

    RMSNorm folded in on either side (rms_t = sqrt(mean_k h[t, k]^2 + eps)):
    ``resid``, ``norm_w``, ``out_partials``: the product is added to the float32 residual
    stream ``resid`` [M, N] in place, ``out`` (bfloat16) becomes resid * norm_w, and
    out_partials [ceil(N / 16), 16] float32 gets the sums of resid^2 over each 16 columns.
    ``in_partials`` (+ ``hidden``, ``eps``): x is such an unnormalised resid * norm_w and
    in_partials its partial sums; row t of the result is divided by rms_t."""
    M, K = x.shape
    N = out.shape[1]
    if w.shape != ((2 * N, K) if gated else (N, K)) or out.shape[0] != M or not out.is_contiguous():
        raise KernelError("gemm_small_m: shapes do not fit")
    if gated:
        if out.dtype != torch.bfloat16:
            raise KernelError("gemm_small_m: the gated product writes bfloat16")
        mode = 2
    else:
        mode = 1 if out.dtype == torch.float32 else 0
        if out.dtype not in (torch.float32, torch.bfloat16):
            raise KernelError("gemm_small_m: out must be bfloat16 or float32")
    in_tiles = 0
    if in_partials is not None:
        if in_partials.dtype != torch.float32 or in_partials.dim() != 2 or in_partials.shape[1] != 16 \
                or not in_partials.is_contiguous() or hidden <= 0:
            raise KernelError("gemm_small_m: in_partials must be contiguous float32 [tiles, 16] with the hidden size given")
        in_tiles = in_partials.shape[0]
    if resid is not None or norm_w is not None or out_partials is not None:
        if gated or out.dtype != torch.bfloat16:
            raise KernelError("gemm_small_m: the residual epilogue writes bfloat16 and is not gated")
        if resid is None or norm_w is None or out_partials is None:
            raise KernelError("gemm_small_m: resid, norm_w and out_partials go together")
        if resid.dtype != torch.float32 or resid.shape != (M, N) or not resid.is_contiguous():
            raise KernelError("gemm_small_m: resid must be contiguous float32 [M, N]")
        if norm_w.dtype != torch.float32 or norm_w.numel() != N or not norm_w.is_contiguous():
            raise KernelError("gemm_small_m: norm_w must be contiguous float32 [N]")
        if out_partials.dtype != torch.float32 or not out_partials.is_contiguous() \
                or out_partials.numel() < -(-N // 16) * 16:
            raise KernelError("gemm_small_m: out_partials must be contiguous float32 [ceil(N / 16), 16]")
        mode = 3
    _cuda(w, out, in_partials, resid, norm_w, out_partials)
    _check(lib().gg_gemm_small_m_fused(_p(x), ctypes.c_longlong(x.stride(0)), _p(w), _p(out), M, N, K, mode,
                                       _p(in_partials), in_tiles, int(hidden), ctypes.c_float(eps),
                                       _p(resid), _p(norm_w), _p(out_partials), _stream()))


_TC_STATUS = {}
tc_launched = False       # a tcgen05 product was launched since the status word was last checked


def tc_status(device) -> torch.Tensor:
    """The status word gemm_tc writes when one of its bounded waits runs out (0 = fine)."""
    key = torch.device(device).index or 0
    if key not in _TC_STATUS:
        _TC_STATUS[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _TC_STATUS[key]


def check_tc_status(device) -> None:
    """Raise if a tensor-core product gave up on a wait since the last check (synchronises)."""
    st = tc_status(device)
    code = int(st.item())
    if code:
        st.zero_()
        raise KernelError(f"gemm_tc gave up waiting on a barrier (code {code}); its output is not valid")


def tc_ok(x: torch.Tensor, w: torch.Tensor, out_cols: int) -> bool:
    """Whether out = x @ w^T can go through gemm_tc."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_cuda and x.shape[0] > 0
            and x.shape[1] % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and w.is_contiguous()
            and out_cols % 2 == 0)


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gated: bool = False,
            pair: bool = False) -> None:
    """out[M, N] = x[M, K] @ w[N, K]^T on tcgen05 (bfloat16 in, float32 accumulate in tensor
    memory); out bfloat16 or float32.  ``gated``: w is [2N, K] (gate rows, then up rows) and
    out = silu(x Wg^T) * (x Wu^T) in bfloat16.  ``pair``: the kernel in which two CTAs on two
    SMs share a 256 x 256 tile (cta_group::2)."""
    M, K = x.shape
    N = out.shape[1]
    if w.shape != ((2 * N, K) if gated else (N, K)) or out.shape[0] != M or not out.is_contiguous():
        raise KernelError("gemm_tc: shapes do not fit")
    if gated and out.dtype != torch.bfloat16:
        raise KernelError("gemm_tc: the gated product writes bfloat16")
    if out.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError("gemm_tc: out must be bfloat16 or float32")
    mode = 2 if gated else (1 if out.dtype == torch.float32 else 0)
    global tc_launched
    tc_launched = True
    fn = lib().gg_gemm_tc2 if pair else lib().gg_gemm_tc
    _check(fn(_p(x), ctypes.c_longlong(x.stride(0)), _p(w), _p(out), M, N, K, mode,
              _p(tc_status(x.device)), _stream()))


MID_M = 64            # most tokens gemm_mid_m takes


def mid_m_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether out = x @ w^T can go through gemm_mid_m."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_cuda
            and 0 < x.shape[0] <= MID_M and x.shape[1] % 8 == 0 and x.stride(1) == 1
            and x.stride(0) % 8 == 0 and w.is_contiguous())


_MID_M_PLANS = {}


def mid_m_plan(M: int, N: int, K: int, gated: bool, device=None):
    """How gemm_mid_m cuts out[M, N] = x[M, K] @ w^T on the current device: (S, boxes, box_rows,
    slabs, ctas_per_sm, ctas_at_once).  It launches S * slabs CTAs."""
    key = (torch.device(device).index if device is not None else torch.cuda.current_device(), M <= 32, N, K, gated)
    plan = _MID_M_PLANS.get(key)
    if plan is None:
        buf = (ctypes.c_int * 6)()
        with torch.cuda.device(key[0]):
            _check(lib().gg_gemm_mid_m_plan(M, N, K, 2 if gated else 0, buf))
        plan = _MID_M_PLANS[key] = tuple(buf)
    return plan


def gemm_mid_m(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gated: bool = False) -> None:
    """out[M, N] = x[M, K] @ w[N, K]^T for M <= 64 on tcgen05 with the operands swapped (rows
    of w on the M side of the instruction, tokens on its N side), the rows of w cut into slabs
    so that the CTAs fill the machine evenly, and K split over a thread-block cluster where the
    slabs are few; out bfloat16 or float32.  ``gated``: w is [2N, K] (gate rows, then up rows)
    and out = silu(x Wg^T) * (x Wu^T) in bfloat16."""
    M, K = x.shape
    N = out.shape[1]
    if w.shape != ((2 * N, K) if gated else (N, K)) or out.shape[0] != M or not out.is_contiguous():
        raise KernelError("gemm_mid_m: shapes do not fit")
    if gated and out.dtype != torch.bfloat16:
        raise KernelError("gemm_mid_m: the gated product writes bfloat16")
    if out.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError("gemm_mid_m: out must be bfloat16 or float32")
    mode = 2 if gated else (1 if out.dtype == torch.float32 else 0)
    global tc_launched
    tc_launched = True
    _check(lib().gg_gemm_mid_m(_p(x), ctypes.c_longlong(x.stride(0)), _p(w), _p(out), M, N, K, mode,
                               _p(tc_status(x.device)), _stream()))


def gemm_tc_withheld(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """Self-test of gemm_tc's bounded waits: launches it with its loads withheld.  The kernel
    gives up after about a second, sets the status word and returns (check_tc_status raises)."""
    M, K = x.shape
    global tc_launched
    tc_launched = True
    _check(lib().gg_gemm_tc_withheld(_p(x), ctypes.c_longlong(x.stride(0)), _p(w), _p(out), M, out.shape[1], K,
                                     _p(tc_status(x.device)), _stream()))


def pack_decode_step(host, offsets, G: int, B: int, Bp: int, used: int, page_size: int, tokens, token_src,
                     state_slots, context_after, tables) -> None:
    """Fill the packed int32 step buffer ``host`` (a numpy view) for a step of single decoded
    tokens: native code over flat numpy arrays (csrc/host_pack.cu).  ``offsets``: int32 array
    of the buffer's array offsets, ``tables``: per group the cache manager's [state slot,
    logical page] int32 table."""
    import numpy as np
    for a in (host, offsets, tokens, token_src, state_slots, context_after, *tables):
        if a.dtype != np.int32 or not a.flags["C_CONTIGUOUS"]:
            raise KernelError("pack_decode_step: arguments must be contiguous int32 arrays")
    ptrs = (ctypes.c_void_p * max(G, 1))(*[t.ctypes.data for t in tables])
    widths = (ctypes.c_int * max(G, 1))(*[t.shape[1] for t in tables])
    vp = lambda a: ctypes.c_void_p(a.ctypes.data)
    _check(lib().gg_pack_decode_step(vp(host), vp(offsets), G, B, Bp, used, page_size, vp(tokens), vp(token_src),
                                     vp(state_slots), vp(context_after), ptrs, widths), 0)


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = first index of the maximum of logits[r, :] (float32 [R, V])."""
    _cuda(logits, out)
    R, V = logits.shape
    if logits.dtype != torch.float32 or out.dtype != torch.int32:
        raise KernelError("argmax: logits float32, out int32")
    _check(lib().gg_argmax(_p(logits), R, V, _p(out), _stream()))


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: Optional[torch.Tensor],
           top_p: Optional[torch.Tensor], seeds: torch.Tensor, draw_index: torch.Tensor,
           out: torch.Tensor) -> None:
    """Per row: greedy if temperature <= 1e-9, else top-k / top-p / seeded categorical."""
    _cuda(logits, temperature, top_k, top_p, seeds, draw_index, out)
    R, V = logits.shape
    if logits.dtype != torch.float32 or out.dtype != torch.int32 or temperature.dtype != torch.float32:
        raise KernelError("sample: logits/temperature float32, out int32")
    if seeds.dtype != torch.int64 or draw_index.dtype != torch.int64:
        raise KernelError("sample: seeds and draw indices must be int64")
    _check(lib().gg_sample(_p(logits), R, V, _p(temperature), _p(top_k), _p(top_p), _p(seeds),
                           _p(draw_index), _p(out), _stream()))
