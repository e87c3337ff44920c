"""Arrangements of a layer's parts.  "pre_norm" is the reference's run_layer
(kernels/gollmgo_model.cu:551-792): x += mixer(norm(x)); x += ffn(norm(x)), the
residual stream x in float32.

Each residual add is fused into the norm that follows it, so a block takes the
residual and a pending delta (what the previous block still owes the residual)
and returns its own pending delta.
"""
from __future__ import annotations

import torch

from .linear import NextNorm, NormedRows
from .registry import register_block


class PreNormBlock:
    """forward(resid, delta, ...) -> the delta this block still owes the residual.

    In steps of a few tokens the two residual adds and norms move into the products around
    them where the parts offer it (the optional protocol of parts/linear.py: a part's
    ``takes_normed_rows(T)`` / ``fuses_next_norm(T)`` and a norm's ``rms_weight_eps()``):
    the mixer's last product adds to the residual and prepares the second norm's input for
    the feed-forward's first product, and the feed-forward's last product does the same for
    the first norm of the block that runs next, if that block ``takes_normed_rows`` too.  The
    delta handed on is then a NormedRows: the add is done and the norm's input is ready."""

    chains_norms = True          # forward takes next_block= and may return or receive NormedRows

    def __init__(self, layer_spec, mixer, feed_forward, mixer_norm, ffn_norm, ctx):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.ffn_norm = mixer_norm, ffn_norm
        self.ctx = ctx
        self.hidden = mixer_norm.size
        ctx.workspace.reserve("normed", ctx.max_tokens * self.hidden, ctx.act_dtype)
        ctx.workspace.reserve("norm_partials", -(-self.hidden // 16) * 16, torch.float32)

    @staticmethod
    def _can(part, what, T):
        f = getattr(part, what, None)
        return bool(f and f(T))

    def takes_normed_rows(self, T):
        """Whether the block before may hand this one its first norm's input as NormedRows."""
        return hasattr(self.mixer_norm, "rms_weight_eps") and self._can(self.mixer, "takes_normed_rows", T)

    def _next_norm(self, norm, resid, T):
        w, eps = norm.rms_weight_eps()
        ws = self.ctx.workspace
        return NextNorm(resid, w, eps, ws.get("normed", T, self.hidden),
                        ws.get("norm_partials", -(-self.hidden // 16), 16))

    def forward(self, resid, delta, batch, cache, writes_cache=True, next_block=None):
        T = resid.shape[0]
        if isinstance(delta, NormedRows):
            h = delta                                   # the block before did the add and prepared the norm
        else:
            h = self.ctx.workspace.get("normed", T, self.hidden)
            self.mixer_norm.add_norm(resid, delta, h)
        if (hasattr(self.ffn_norm, "rms_weight_eps") and self._can(self.mixer, "fuses_next_norm", T)
                and self._can(self.feed_forward, "takes_normed_rows", T)):
            h = self.mixer.forward(h, batch, cache, writes_cache, then=self._next_norm(self.ffn_norm, resid, T))
        else:
            a = self.mixer.forward(h, batch, cache, writes_cache)
            h = self.ctx.workspace.get("normed", T, self.hidden)
            self.ffn_norm.add_norm(resid, a, h)
        nxt = next_block
        if (nxt is not None and getattr(nxt, "chains_norms", False) and nxt.takes_normed_rows(T)
                and nxt.hidden == self.hidden and self._can(self.feed_forward, "fuses_next_norm", T)):
            return self.feed_forward.forward(h, batch, then=self._next_norm(nxt.mixer_norm, resid, T))
        return self.feed_forward.forward(h, batch)


register_block("pre_norm", PreNormBlock)
