"""The SiLU-gated feed-forward: down( silu(x Wg^T) * (x Wu^T) ), no biases
(kernels/gollmgo_model.cu:746-776, kernels/gollmgo_ops.cu:361-374).  Gate and up
weights are stacked so one product makes both.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights import WeightSpec
from .linear import NormedRows, fuses_norms, linear, use_mid_m, use_tc
from .registry import register_feed_forward


class GatedMLP:
    """params: hidden_size, intermediate_size, activation ("silu")."""

    def __init__(self, spec, ctx):
        self.ctx = ctx
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        act = spec.get("activation", "silu")
        if act != "silu":
            raise ValueError(f"activation {act!r} is not supported (known: silu)")
        ws, T = ctx.workspace, ctx.max_tokens
        ws.reserve("gate_up", T * 2 * self.inter, ctx.act_dtype)
        ws.reserve("ffn_act", T * self.inter, ctx.act_dtype)
        ws.reserve("ffn_out", T * self.hidden, ctx.act_dtype)
        self.w_gate_up = None
        self.w_down = None

    def weights(self):
        return {"gate_proj.weight": WeightSpec((self.inter, self.hidden)),
                "up_proj.weight": WeightSpec((self.inter, self.hidden)),
                "down_proj.weight": WeightSpec((self.hidden, self.inter))}

    def load(self, get):
        g, u = get("gate_proj.weight"), get("up_proj.weight")
        dt = torch.float32 if torch.float32 in (g.dtype, u.dtype) else g.dtype
        self.w_gate_up = torch.cat([g.to(dt), u.to(dt)], dim=0).contiguous()
        self.w_down = get("down_proj.weight").contiguous()

    # the optional protocol of parts/linear.py: the first product can take a norm's unnormalised
    # input, the last one can do the residual add and prepare the next norm
    def takes_normed_rows(self, num_tokens):
        return fuses_norms(num_tokens, self.w_gate_up, self.ctx.act_dtype)

    def fuses_next_norm(self, num_tokens):
        return fuses_norms(num_tokens, self.w_down, self.ctx.act_dtype)

    def forward(self, x, batch, then=None):
        T = x.shape[0]
        ws = self.ctx.workspace
        a = ws.get("ffn_act", T, self.inter)
        if isinstance(x, NormedRows):
            ops.gemm_small_m(x.scaled, self.w_gate_up, a, gated=True, in_partials=x.partials,
                             hidden=x.hidden, eps=x.eps)
        elif ops.small_m_ok(x, self.w_gate_up):
            ops.gemm_small_m(x, self.w_gate_up, a, gated=True)       # product and activation in one
        elif use_mid_m(x, self.w_gate_up, gated=True):
            ops.gemm_mid_m(x, self.w_gate_up, a, gated=True)          # the same for a few dozen tokens
        elif use_tc(x, self.w_gate_up, self.inter, True):
            ops.gemm_tc(x, self.w_gate_up, a, gated=True, pair=True)  # the same, on tcgen05 (CTA pairs)
        else:
            gu = ws.get("gate_up", T, 2 * self.inter)
            linear(x, self.w_gate_up, gu)
            ops.silu_mul(gu, a)
        y = ws.get("ffn_out", T, self.hidden)
        return linear(a, self.w_down, y, then)


register_feed_forward("gated_mlp", GatedMLP)
