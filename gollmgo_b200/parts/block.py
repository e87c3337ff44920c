"""Arrangements of a layer's parts.  "pre_norm" is the reference's run_layer
(kernels/gollmgo_model.cu:551-792): x += mixer(norm(x)); x += ffn(norm(x)), the
residual stream x in float32.

Each residual add is fused into the norm that follows it, so a block takes the
residual and a pending delta (what the previous block still owes the residual)
and returns its own pending delta.
"""
from __future__ import annotations

from .registry import register_block


class PreNormBlock:
    def __init__(self, layer_spec, mixer, feed_forward, mixer_norm, ffn_norm, ctx):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.ffn_norm = mixer_norm, ffn_norm
        self.ctx = ctx
        self.hidden = mixer_norm.size
        ctx.workspace.reserve("normed", ctx.max_tokens * self.hidden, ctx.act_dtype)

    def forward(self, resid, delta, batch, cache, writes_cache=True):
        T = resid.shape[0]
        h = self.ctx.workspace.get("normed", T, self.hidden)
        self.mixer_norm.add_norm(resid, delta, h)
        a = self.mixer.forward(h, batch, cache, writes_cache)
        self.ffn_norm.add_norm(resid, a, h)
        return self.feed_forward.forward(h, batch)


register_block("pre_norm", PreNormBlock)
