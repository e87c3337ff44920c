"""What a model is made of, as data.

An architecture turns its typed configuration into a ``ModelSpec``: one
``LayerSpec`` per layer (which mixer, which feed-forward, which norms, arranged
by which block, each with its sizes and constants as parameters) and a run
order.  The generic ``DecoderModel`` builds the parts named here from the parts
registry; no part knows which model it is in.

The run order is a list of ``RunEntry``.  An entry names the layer to run and the
cache entry it uses; a layer may be named twice (each occurrence with a cache
entry of its own), and an entry with ``writes_cache=False`` reads the cache that
another entry wrote instead of writing its own.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """A part by registry name with its parameters (sizes, constants)."""
    kind: str
    params: Dict[str, object] = field(default_factory=dict)

    def __getitem__(self, key):
        return self.params[key]

    def get(self, key, default=None):
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    block: PartSpec                    # arrangement, e.g. "pre_norm"
    mixer: PartSpec                    # e.g. "attention"
    feed_forward: PartSpec             # e.g. "gated_mlp"
    mixer_norm: PartSpec               # norm before the mixer
    ffn_norm: PartSpec                 # norm before the feed-forward
    # checkpoint names: prefix of the mixer's and feed-forward's tensors, full
    # names of the two norm weights
    mixer_prefix: str = ""
    ffn_prefix: str = ""
    mixer_norm_name: str = ""
    ffn_norm_name: str = ""


@dataclass(frozen=True)
class RunEntry:
    layer: int
    cache: int                         # index of the cache entry this occurrence uses
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: Tuple[LayerSpec, ...]
    run_order: Tuple[RunEntry, ...]
    final_norm: PartSpec
    tie_embeddings: bool
    embed_name: str
    final_norm_name: str
    head_name: str
    max_positions: int
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    # a position encoding that acts on the embedded tokens, before the first layer (a table of
    # learned positions, say), with the prefix of its checkpoint tensors; None = the layers'
    # mixers do all the position encoding there is (rotary: inside attention)
    embed_position: Optional[PartSpec] = None
    embed_position_prefix: str = ""

    @property
    def num_cache_entries(self) -> int:
        return 1 + max((e.cache for e in self.run_order), default=-1)
