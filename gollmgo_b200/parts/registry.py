"""Registries of part kinds: mixers, feed-forwards, norms, position encodings and
block arrangements.  ``register_*`` adds a kind under a name; a ``PartSpec`` with
that ``kind`` is then built by ``build_*``.  A test or a user can register a part
of their own without touching this package.

Interfaces (``ctx`` is a ``BuildContext``; tensors of activations are
``[tokens, width]`` in ``ctx.act_dtype``):

norm            cls(spec, ctx)
                  .weights() -> {local name: WeightSpec}     ("" = the norm's one tensor)
                  .load(get)                                  get(local name) -> tensor
                  .add_norm(resid, delta, out, rows=None, write_back=True)
position        cls(spec, ctx)
                  .rope_table() -> float64 tensor [rot/2] or None   (fused in the cache-write kernel)
                  .interleaved: bool
                  .apply(qkv, batch, nh, nkv, d)              optional: rewrite the q and k heads of
                                                              qkv [T, (nh+2nkv)*d] in place (positions in
                                                              batch.positions) before k, v go to the cache
                a position encoding named in ModelSpec.embed_position acts on the embedded tokens
                instead and offers
                  .weights(), .load(get)                      its tensors, under ModelSpec.embed_position_prefix
                  .add_to_embedding(resid, batch)             resid [T, hidden] float32, in place
mixer           cls(spec, ctx)
                  .cache_need() -> PagedKVNeed | FixedStateNeed | None
                  .weights(), .load(get)
                  .forward(x, batch, cache, writes_cache) -> tensor [T, hidden]
                  .query_tiles() -> [QueryTiles]              optional: index lists over the query rows of
                                                              prompt portions that every batch should hold
                                                              for it (batch.tiles[need])
                  .step_tags(facts) -> tuple of str           optional (any part): tags of a step, from the
                                                              StepFacts known before its batch is built; the
                                                              runner captures steps of different tags
                                                              separately and sets batch.tags
feed-forward    cls(spec, ctx)
                  .weights(), .load(get)
                  .forward(x, batch) -> tensor [T, hidden]
block           cls(layer_spec, mixer, feed_forward, mixer_norm, ffn_norm, ctx)
                  .forward(resid, delta, batch, cache, writes_cache) -> pending delta
"""
from __future__ import annotations

from typing import Callable, Dict

_KINDS = ("norm", "position", "mixer", "feed_forward", "block")
_REG: Dict[str, Dict[str, Callable]] = {k: {} for k in _KINDS}


def _register(family: str, name: str, cls: Callable) -> None:
    _REG[family][name] = cls


def _build(family: str, spec, *args):
    try:
        cls = _REG[family][spec.kind]
    except KeyError:
        raise KeyError(f"no {family} named {spec.kind!r} is registered; known: "
                       f"{sorted(_REG[family])}") from None
    return cls(spec, *args)


def register_norm(name, cls): _register("norm", name, cls)
def register_position(name, cls): _register("position", name, cls)
def register_mixer(name, cls): _register("mixer", name, cls)
def register_feed_forward(name, cls): _register("feed_forward", name, cls)
def register_block(name, cls): _register("block", name, cls)


def build_norm(spec, ctx): return _build("norm", spec, ctx)
def build_position(spec, ctx): return _build("position", spec, ctx)
def build_mixer(spec, ctx): return _build("mixer", spec, ctx)
def build_feed_forward(spec, ctx): return _build("feed_forward", spec, ctx)


def build_block(layer_spec, mixer, feed_forward, mixer_norm, ffn_norm, ctx):
    try:
        cls = _REG["block"][layer_spec.block.kind]
    except KeyError:
        raise KeyError(f"no block named {layer_spec.block.kind!r} is registered; known: "
                       f"{sorted(_REG['block'])}") from None
    return cls(layer_spec, mixer, feed_forward, mixer_norm, ffn_norm, ctx)


def known(family: str):
    return sorted(_REG[family])
