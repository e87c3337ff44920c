"""Position encodings.  "rope": rotary, inverse frequencies from theta with the
optional llama3 or linear scaling of config.json's ``rope_scaling``; "none".

The reference rotates with f_p = theta^(-2p/d), theta fixed at 10000 and no
scaling (kernels/gollmgo_ops.cu:337, kernels/gollmgo_model.cu:603).  The table is
built once on the host in float64 and handed to the kernel that rotates q and k
and writes the cache.
"""
from __future__ import annotations

import math

import torch

from .registry import register_position


def inverse_frequencies(rot: int, theta: float, scaling) -> torch.Tensor:
    p = torch.arange(0, rot, 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(theta, dtype=torch.float64), -p / rot)
    if scaling is None:
        return f
    if scaling.rope_type == "linear":
        return f / scaling.factor
    if scaling.rope_type == "llama3":
        orig = float(scaling.original_max_position_embeddings)
        lo_wl = orig / scaling.low_freq_factor        # longer than this: slowed by factor
        hi_wl = orig / scaling.high_freq_factor       # shorter than this: kept
        wl = 2.0 * math.pi / f
        smooth = (orig / wl - scaling.low_freq_factor) / (scaling.high_freq_factor - scaling.low_freq_factor)
        blended = (1.0 - smooth) * f / scaling.factor + smooth * f
        return torch.where(wl < hi_wl, f, torch.where(wl > lo_wl, f / scaling.factor, blended))
    raise ValueError(f"rope scaling {scaling.rope_type!r} is not supported")


class RotaryEncoding:
    """params: head_dim, theta, scaling (config.RopeScaling or None), interleaved,
    rotary_dim (defaults to head_dim)."""

    def __init__(self, spec, ctx):
        self.head_dim = int(spec["head_dim"])
        self.rot = int(spec.get("rotary_dim") or self.head_dim)
        if self.rot % 2 or self.rot > self.head_dim:
            raise ValueError(f"rotary width {self.rot} must be even and at most {self.head_dim}")
        self.interleaved = bool(spec.get("interleaved", False))
        self._table = inverse_frequencies(self.rot, float(spec["theta"]), spec.get("scaling")) \
            .to(ctx.device).contiguous()

    def rope_table(self):
        return self._table


class NoPositionEncoding:
    interleaved = False

    def __init__(self, spec, ctx):
        pass

    def rope_table(self):
        return None


register_position("rope", RotaryEncoding)
register_position("none", NoPositionEncoding)
