"""Matrix products of the model: out = x @ w^T.  Steps of up to 16 tokens in
bfloat16 go through this package's weight-streaming kernel (csrc/gemm_small_m.cu),
the gated feed-forward product of longer steps through its tcgen05 kernel
(csrc/gemm_tc.cu), the rest through the vendor library, as in the reference
(cublasGemmEx with float32 accumulation: kernels/gollmgo_model.cu:143-169).

In the float32 mode the product is a true float32 one: the TF32 matrix mode and
reduced-precision accumulation are switched off for the process by
``set_matmul_precision``.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops


def set_matmul_precision() -> None:
    """No TF32 for float32 products, no bfloat16 accumulation across split-K."""
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.set_float32_matmul_precision("highest")
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False


import os

# Which kernel multiplies more than 16 tokens: "tc" = this package's tcgen05 kernel for
# every product, "lib" = the vendor library for every product, "auto" (default) = the
# tcgen05 kernel where it is measured to be at least level (the gated product, whose
# activation it fuses), the library elsewhere.
GEMM_POLICY = os.environ.get("GOLLMGO_B200_GEMM", "auto")


TC_MIN_TOKENS = 1024     # below this the tcgen05 kernel has too few tiles to fill the machine


# Steps of 17 to MID_M_TOKENS tokens use this package's swapped-operand tcgen05 kernel
# (csrc/gemm_mid_m.cu), which takes up to 64.  Measured on whole decode steps of the
# Llama-3.1-8B shape: 2.7 % faster than the vendor library at 24 tokens, level at 32, 3 %
# slower at 64 (its 224 row slabs of the gated product fill 296 places unevenly).
MID_M_TOKENS = int(os.environ.get("GOLLMGO_B200_GEMM_MID_TOKENS", "32"))
# Up to MID_M_SPLIT_TOKENS tokens it still takes the products with so few rows of W that it
# splits K eight ways over a cluster (the o and down products of that shape: 12.6 and 25.9 us
# against the library's 15.5 and 27.0 at 64 tokens).
MID_M_SPLIT_TOKENS = int(os.environ.get("GOLLMGO_B200_GEMM_MID_SPLIT_TOKENS", "64"))
_NUM_SMS = {}


def _num_sms(device) -> int:
    n = _NUM_SMS.get(device)
    if n is None:
        n = _NUM_SMS[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return n


def use_mid_m(x: torch.Tensor, w: torch.Tensor) -> bool:
    if GEMM_POLICY == "lib":
        return False
    T = x.shape[0]
    if not x.is_cuda:
        return False
    slabs, places = -(-w.shape[0] // 128), 2 * _num_sms(x.device)
    if slabs > places:          # several rounds of CTAs (an LM head): the library is ahead, 167 vs 188 us at 32 tokens
        return False
    if T > MID_M_TOKENS and not (T <= MID_M_SPLIT_TOKENS and slabs * 8 <= places):
        return False
    return ops.mid_m_ok(x, w)


def use_tc(x: torch.Tensor, w: torch.Tensor, out_cols: int, gated: bool) -> bool:
    if GEMM_POLICY == "lib" or not ops.tc_ok(x, w, out_cols):
        return False
    return GEMM_POLICY == "tc" or (gated and x.shape[0] >= TC_MIN_TOKENS)


# Steps of a few tokens: the residual add and the RMSNorm between two products are done by
# the products themselves (csrc/gemm_small_m.cu) instead of by a kernel between them.
FUSE_NORMS = os.environ.get("GOLLMGO_B200_FUSE_NORM", "1") != "0"


class NextNorm:
    """What the last product of a mixer or feed-forward is asked to do with its result y
    instead of returning it: resid += y, and leave the input of the norm (weight, eps) that
    follows as NormedRows in the buffers ``scaled`` [T, hidden] and ``partials``."""

    def __init__(self, resid, weight, eps, scaled, partials):
        self.resid, self.weight, self.eps = resid, weight, eps
        self.scaled, self.partials = scaled, partials


class NormedRows:
    """A norm's output that is not divided by the root mean square yet: ``scaled`` is
    resid * weight in bfloat16, ``partials[tile, t]`` the sums of resid[t]^2 over slices of
    the hidden size.  The product that takes it as x multiplies row t of its result by
    rsqrt(sum(partials[:, t]) / hidden + eps): one factor per token, so the same as
    normalising x first."""

    def __init__(self, scaled, partials, hidden, eps):
        self.scaled, self.partials, self.hidden, self.eps = scaled, partials, hidden, eps

    @property
    def shape(self):
        return self.scaled.shape


def fuses_norms(num_tokens: int, w: torch.Tensor, act_dtype: torch.dtype) -> bool:
    """Whether a product with weight w of a step of num_tokens tokens can take NormedRows
    as x, or do what a NextNorm asks."""
    return (FUSE_NORMS and w is not None and w.is_cuda and 0 < num_tokens <= ops.SMALL_M
            and act_dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous()
            and w.shape[1] % 8 == 0)


def linear(x, w: torch.Tensor, out: torch.Tensor, then: Optional[NextNorm] = None):
    """out[T, N] = x[T, K] @ w[N, K]^T, rounded to out's dtype.  A weight stored in
    float32 is multiplied in float32 even when the activations are bfloat16.
    x may be NormedRows and ``then`` a NextNorm where fuses_norms() holds (the caller
    checks); with ``then`` the result is the NormedRows of the next norm, not out."""
    if isinstance(x, NormedRows) or then is not None:
        rows = x if isinstance(x, NormedRows) else None
        xt = rows.scaled if rows else x
        kw = dict(in_partials=rows.partials, hidden=rows.hidden, eps=rows.eps) if rows else {}
        if then is None:
            ops.gemm_small_m(xt, w, out, **kw)
            return out
        ops.gemm_small_m(xt, w, then.scaled, resid=then.resid, norm_w=then.weight, out_partials=then.partials, **kw)
        return NormedRows(then.scaled, then.partials, then.scaled.shape[1], then.eps)
    if ops.small_m_ok(x, w) and out.is_contiguous():
        ops.gemm_small_m(x, w, out)          # a few tokens: the weight-streaming kernel
    elif use_mid_m(x, w) and out.is_contiguous():
        ops.gemm_mid_m(x, w, out)            # a few dozen tokens: the same on tcgen05, operands swapped
    elif out.is_contiguous() and use_tc(x, w, out.shape[1], False):
        ops.gemm_tc(x, w, out)
    elif w.dtype == x.dtype and out.dtype == x.dtype:
        torch.mm(x, w.t(), out=out)
    elif w.dtype == x.dtype and out.dtype == torch.float32:
        out.copy_(torch.mm(x, w.t(), out_dtype=torch.float32))
    else:
        out.copy_(torch.mm(x.to(torch.float32), w.to(torch.float32).t()))
    return out
