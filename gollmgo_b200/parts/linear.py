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
# (csrc/gemm_mid_m.cu) for every product that it runs as one round of CTAs; a product of
# several rounds (an LM head) stays with the vendor library (201 against 182 us at 64 tokens).
# The threshold is from whole decode steps of the Llama-3.1-8B shape (ms per step, own kernel
# for all four products of a layer / library for all): 32 sequences 4.97 / 5.20, 40: 5.45 /
# 5.60, 48: 5.54 / 5.56, 64: 6.86 / 6.75.  Timed alone, back to back, the own kernel is ahead
# at 64 tokens as well (qkv 14.6 us against 15.5, o 11.8 / 15.4, gate_up with the activation
# 42.6 / 45.0 + 2.5, down 25.1 / 27.0): a launch overlaps the end of the same kernel before it
# better than the end of the attention, so the step decides, not the loop.
MID_M_TOKENS = int(os.environ.get("GOLLMGO_B200_GEMM_MID_TOKENS", "48"))
# The products whose K is split eight ways (o and down of that shape) may go further.
MID_M_SPLIT_TOKENS = int(os.environ.get("GOLLMGO_B200_GEMM_MID_SPLIT_TOKENS", "48"))


def use_mid_m(x: torch.Tensor, w: torch.Tensor, gated: bool = False) -> bool:
    if GEMM_POLICY == "lib" or not x.is_cuda or not ops.mid_m_ok(x, w):
        return False
    T = x.shape[0]
    N = w.shape[0] // 2 if gated else w.shape[0]
    S, _, _, slabs, _, at_once = ops.mid_m_plan(T, N, x.shape[1], gated, x.device)
    if T > MID_M_TOKENS and not (T <= MID_M_SPLIT_TOKENS and S == 8):
        return False
    return S * slabs <= at_once


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
