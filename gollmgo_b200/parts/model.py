"""The generic decoder: embedding, the layers in run order, final norm, LM head.

Built from a ``ModelSpec`` alone.  Data flow per step (reference:
kernels/gollmgo_model.cu:796-858 and run_layer): ids -> float32 residual stream
-> blocks -> rows whose logits are wanted -> final norm -> head product ->
float32 logits.  The reference computes the head for every token of a prompt;
here only the wanted rows reach the final norm and the head.
"""
from __future__ import annotations

from typing import Callable, Dict, List

import torch

from ..config import read_config_json, resolve_architecture
from ..csrc import ops
from ..weights import WeightSpec
from .context import BuildContext
from .linear import linear
from .registry import build_block, build_feed_forward, build_mixer, build_norm, build_position
from .spec import ModelSpec


def _prefixed(prefix: str, weights: Dict[str, WeightSpec], single_name: str = "") -> Dict[str, WeightSpec]:
    return {(single_name if local == "" else prefix + local): spec for local, spec in weights.items()}


def spec_manifest(spec: ModelSpec, parts=None, embed_position=None) -> Dict[str, WeightSpec]:
    """Checkpoint tensors the model expects.  ``parts`` = per layer
    (mixer, feed_forward, mixer_norm, ffn_norm) if already built."""
    m: Dict[str, WeightSpec] = {spec.embed_name: WeightSpec((spec.vocab_size, spec.hidden_size))}
    for ls, (mixer, ff, n1, n2) in zip(spec.layers, parts):
        m.update(_prefixed(ls.mixer_prefix, mixer.weights()))
        m.update(_prefixed(ls.ffn_prefix, ff.weights()))
        m.update(_prefixed("", n1.weights(), ls.mixer_norm_name))
        m.update(_prefixed("", n2.weights(), ls.ffn_norm_name))
    m[spec.final_norm_name] = WeightSpec((spec.hidden_size,))
    if embed_position is not None:
        m.update(_prefixed(spec.embed_position_prefix, embed_position.weights()))
    m[spec.head_name] = WeightSpec((spec.vocab_size, spec.hidden_size), optional=spec.tie_embeddings)
    return m


class DecoderModel:
    def __init__(self, spec: ModelSpec, ctx: BuildContext):
        self.spec, self.ctx = spec, ctx
        self.parts = []
        self.blocks = []
        for ls in spec.layers:
            mixer = build_mixer(ls.mixer, ctx)
            ff = build_feed_forward(ls.feed_forward, ctx)
            n1, n2 = build_norm(ls.mixer_norm, ctx), build_norm(ls.ffn_norm, ctx)
            self.parts.append((mixer, ff, n1, n2))
            self.blocks.append(build_block(ls, mixer, ff, n1, n2, ctx))
        self.final_norm = build_norm(spec.final_norm, ctx)
        self.embed_position = build_position(spec.embed_position, ctx) if spec.embed_position else None
        ws = ctx.workspace
        ws.reserve("residual", ctx.max_tokens * spec.hidden_size, torch.float32)
        ws.reserve("head_in", ctx.max_tokens * spec.hidden_size, ctx.act_dtype)
        self.embed = None
        self.head = None
        self.bad_id = torch.zeros(1, dtype=torch.int32, device=ctx.device) \
            if ctx.device.type == "cuda" else None

    # ------------------------------------------------------------------ weights
    def manifest(self) -> Dict[str, WeightSpec]:
        return spec_manifest(self.spec, self.parts, self.embed_position)

    def load(self, get: Callable[[str], torch.Tensor]) -> None:
        """Bind weights: ``get(name)`` delivers a checkpoint tensor on the device."""
        s = self.spec
        self.embed = get(s.embed_name).contiguous()
        for ls, (mixer, ff, n1, n2) in zip(s.layers, self.parts):
            mixer.load(lambda local, p=ls.mixer_prefix: get(p + local))
            ff.load(lambda local, p=ls.ffn_prefix: get(p + local))
            n1.load(lambda local, n=ls.mixer_norm_name: get(n))
            n2.load(lambda local, n=ls.ffn_norm_name: get(n))
        self.final_norm.load(lambda local: get(s.final_norm_name))
        if self.embed_position is not None:
            self.embed_position.load(lambda local, p=s.embed_position_prefix: get(p + local))
        head = None if s.tie_embeddings else get(s.head_name)
        self.head = self.embed if head is None else head.contiguous()

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        def add(t):
            nonlocal total
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        add(self.embed), add(self.head), add(self.final_norm.weight)
        for mixer, ff, n1, n2 in self.parts:
            for part in (mixer, ff, n1, n2):
                for v in vars(part).values():
                    if isinstance(v, torch.Tensor) and v.dim() >= 1 and v.is_cuda:
                        add(v)
        return total

    # ------------------------------------------------------------------ cache
    def cache_needs(self) -> List[object]:
        """Per cache entry of the run order, what it needs of the cache manager."""
        needs: List[object] = [None] * self.spec.num_cache_entries
        for e in self.spec.run_order:
            need = self.parts[e.layer][0].cache_need()
            if needs[e.cache] is not None and needs[e.cache] != need:
                raise ValueError(f"cache entry {e.cache} is used by layers with different needs")
            needs[e.cache] = need
        return needs

    # ------------------------------------------------------------------ what the parts ask of a step
    def query_tiles(self) -> list:
        """The index lists (QueryTiles) the mixers want in every step's batch."""
        wanted = []
        for mixer, _, _, _ in self.parts:
            for need in getattr(mixer, "query_tiles", lambda: ())():
                if need not in wanted:
                    wanted.append(need)
        return wanted

    def step_tags(self, facts) -> tuple:
        """The step's kind: the tags of every part that offers ``step_tags(facts)``, sorted."""
        tags = set()
        for parts in self.parts:
            for part in parts:
                f = getattr(part, "step_tags", None)
                if f is not None:
                    tags.update(f(facts))
        return tuple(sorted(tags))

    # ------------------------------------------------------------------ forward
    def forward(self, batch, caches) -> torch.Tensor:
        """Run the batch's tokens; return float32 logits [len(logit_rows), vocab].
        ``caches[i]`` is what the cache manager holds for cache entry i."""
        T, H = batch.num_tokens, self.spec.hidden_size
        ws = self.ctx.workspace
        resid = ws.get("residual", T, H)
        ops.embed_gather(batch.token_ids, self.embed, resid, self.bad_id,
                         getattr(batch, "token_src", None), getattr(batch, "prev_tokens", None))
        if self.embed_position is not None:
            self.embed_position.add_to_embedding(resid, batch)
        delta = None
        order = self.spec.run_order
        for i, e in enumerate(order):
            block = self.blocks[e.layer]
            if getattr(block, "chains_norms", False):
                # such a block may fold the first norm of the block that runs next into its last product
                nxt = self.blocks[order[i + 1].layer] if i + 1 < len(order) else None
                delta = block.forward(resid, delta, batch, caches[e.cache], e.writes_cache, next_block=nxt)
            else:
                delta = block.forward(resid, delta, batch, caches[e.cache], e.writes_cache)
        R = batch.num_logit_rows
        logits = torch.empty(R, self.spec.vocab_size, dtype=torch.float32, device=self.ctx.device)
        if R == 0:
            return logits
        h = ws.get("head_in", R, H)
        self.final_norm.add_norm(resid, delta, h, rows=batch.logit_rows, write_back=False)
        linear(h, self.head, logits)
        return logits


def build_model(config_dict: dict, ctx: BuildContext):
    """config.json dict -> (typed config, ModelSpec, DecoderModel) via the registry."""
    arch = resolve_architecture(config_dict)
    cfg = arch.parse(config_dict)
    spec = arch.spec(cfg)
    return cfg, spec, DecoderModel(spec, ctx)


def manifest_for_config(config_dict: dict) -> Dict[str, WeightSpec]:
    """Tensors a checkpoint of this configuration holds (no device needed)."""
    ctx = BuildContext(torch.float32, "cpu", 1, 1, 16)
    return build_model(config_dict, ctx)[2].manifest()
