"""RMSNorm, fused with the residual add that precedes it.

y = x * rsqrt(mean(x^2) + eps) * w in float32 (kernels/gollmgo_ops.cu:593-629);
eps comes from config.json (the reference passes the literal 1e-5:
internal/backend/cuda/model_bridge.go:53).
"""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights import WeightSpec
from .registry import register_norm


class RMSNorm:
    def __init__(self, spec, ctx):
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.ctx = ctx
        self.weight = None

    def weights(self):
        return {"": WeightSpec((self.size,))}

    def load(self, get):
        self.weight = get("").to(torch.float32).contiguous()

    def rms_weight_eps(self):
        """(weight, eps) for a product that folds this norm in (parts/linear.py): only a norm
        that is exactly x * rsqrt(mean(x^2) + eps) * weight may offer this."""
        return self.weight, self.eps

    def add_norm(self, resid, delta, out, rows=None, write_back=True):
        """resid (+= delta); out = norm(resid) * weight.  With ``rows`` only those rows
        are normed (out[i] from resid[rows[i]])."""
        ops.add_rmsnorm(resid, delta, self.weight, out, self.eps, rows, write_back)
        return out


register_norm("rmsnorm", RMSNorm)
