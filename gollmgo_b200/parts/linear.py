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


def use_tc(x: torch.Tensor, w: torch.Tensor, out_cols: int, gated: bool) -> bool:
    if GEMM_POLICY == "lib" or not ops.tc_ok(x, w, out_cols):
        return False
    return GEMM_POLICY == "tc" or (gated and x.shape[0] >= TC_MIN_TOKENS)


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[T, N] = x[T, K] @ w[N, K]^T, rounded to out's dtype.  A weight stored in
    float32 is multiplied in float32 even when the activations are bfloat16."""
    if ops.small_m_ok(x, w) and out.is_contiguous():
        ops.gemm_small_m(x, w, out)          # a few tokens: the weight-streaming kernel
    elif out.is_contiguous() and use_tc(x, w, out.shape[1], False):
        ops.gemm_tc(x, w, out)
    elif w.dtype == x.dtype and out.dtype == x.dtype:
        torch.mm(x, w.t(), out=out)
    elif w.dtype == x.dtype and out.dtype == torch.float32:
        out.copy_(torch.mm(x, w.t(), out_dtype=torch.float32))
    else:
        out.copy_(torch.mm(x.to(torch.float32), w.to(torch.float32).t()))
    return out
