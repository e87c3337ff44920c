"""The attention mixer: q/k/v projections, position encoding, cache write,
grouped-query attention over the paged cache, output projection.

Order of operations follows the reference's run_layer (kernels/gollmgo_model.cu:581-713):
projections without bias, rotation of q and k, write of k and v at this step's
slots, attention over everything the cache holds for the sequence (this step's
tokens included), output projection.  q, k and v come from one product with the
three weights stacked.
"""
from __future__ import annotations

import functools
import math
import os

import torch

from ..cache import PagedKVNeed
from ..csrc import ops
from ..weights import WeightSpec
from .context import QueryTiles
from .linear import fuses_norms, linear
from .registry import build_position, register_mixer

# Which prompt-attention kernel the bfloat16 mode uses: "auto" = the most specialised one that
# takes the sizes (tcgen05 for head sizes 64 and 128 in prompt portions, mma.sync for decode), "mma" = no tcgen05 kernel,
# "general" = only the general kernel.
ATTN_POLICY = os.environ.get("GOLLMGO_B200_ATTN", "auto")
SHORT_PROMPT_KEYS = int(os.environ.get("GOLLMGO_B200_ATTN_SHORT_KEYS", "256"))   # see Attention._few_short_tiles
# Steps of decoded tokens only: rotation and cache write inside the decode attention kernel.
FUSE_DECODE_ROPE = os.environ.get("GOLLMGO_B200_FUSE_ROPE", "1") != "0"
# Decode steps with at least this many times more (token, kv head) pairs than CTAs fit at once
# use the kernel that cuts all tiles into equal ranges (ops.attn_decode_flat); 0 = never.
FLAT_DECODE_FILL = float(os.environ.get("GOLLMGO_B200_FLAT_DECODE_FILL", "1.0"))
MAX_SPLITS = 16
# The index lists over the query rows of prompt portions that the three prompt kernels walk:
# tiles of 16 rows (general kernel, csrc/attention.cu), of 64 (mma.sync, csrc/attention_mma.cu),
# of 128 with the tiles that attend to most keys first (tcgen05, csrc/attention_tc.cu)
TILES_GENERAL, TILES_MMA, TILES_TC = QueryTiles(16), QueryTiles(64), QueryTiles(128, most_keys_first=True)
FORCED_SPLITS = int(os.environ.get("GOLLMGO_B200_DECODE_SPLITS", "0"))   # for measurements: this count, whatever the batch
CTAS_PER_SM = 3            # decode attention CTAs resident on one SM (csrc/attention_mma.cu)
TILE_KEYS = 64             # keys of one tile of the decode kernels
# Into how many slices the context of a decoded token is cut is chosen from the step itself: the
# batch, and the longest context any live request holds, rounded up to a power of two of tiles
# (the attention tags a step with the count it chose, so a captured step is replayed only for
# steps that would choose the same).  The estimate is in microseconds and bytes.  What is
# measured (B200, the decode kernel of csrc/attention_mma.cu) and what is derived:
CTA_STREAM_BYTES_PER_US = 20480.0   # one CTA alone streams a 32 KB tile (64 keys x 128 x k, v x bfloat16) in 1.6 us
HBM_BYTES_PER_US = 6.8e6            # what the kernel streams at best with every CTA busy: no choice gets below bytes / this
SPLIT_OVERHEAD_US = 6.4             # fixed cost with a merge kernel (prologue, combine, merge launch)
CLUSTER_OVERHEAD_US = 3.2           # fixed cost where the slices merge inside a cluster instead
PER_SLICE_US = 0.48                 # what every further slice adds (barriers, partial results to merge)
WAVE_PENALTY_US = 6.4               # every further round of CTAs or clusters, beyond its tiles
CLUSTER_FILL = 0.9         # share of the cluster capacity that one round can count on: clusters are placed
                           # while the kernel before still drains, and a launch that needs every last place
                           # often waits for a second round (measured: a quarter of the launches, 11 us each).
                           # A launch of several rounds anyway fills every place (batch 32: three slices in
                           # two rounds, 52.8 us a layer, against 61.1 for whole contexts on 256 of 444 places)
# Contexts of this many tiles or more (8192 tokens) of so few sequences that even the largest
# cluster per pair leaves places empty may be cut into up to MAX_SPLITS_MANY slices, merged by a
# kernel of their own.  One sequence at 32768 tokens: 8 slices in a cluster are 64 CTAs for
# 134 MB of cache a layer (87 us); 32 slices and a merge kernel are 256 CTAs.
MANY_SLICES_FROM_TILES = 128
MAX_SPLITS_MANY = 64
MAX_TILES = 1024


def context_tiles(max_context: int, window=None) -> int:
    """Tiles of the longest context (or of the window, if shorter), rounded up to a power of
    two: the sizes the choice of slices is made for."""
    keys = max(1, int(max_context))
    if window:
        keys = min(keys, int(window) + TILE_KEYS)
    tiles = -(-keys // TILE_KEYS)
    return min(MAX_TILES, 1 << (tiles - 1).bit_length())


@functools.lru_cache(maxsize=4096)
def _decode_splits(n_dec, ctas_per_split, num_sms, cluster_capacity, tiles, tile_bytes, forced):
    if forced > 0:
        return forced
    slots = CTAS_PER_SM * num_sms
    ctas = max(1, n_dec * ctas_per_split)
    tile_us = tile_bytes / CTA_STREAM_BYTES_PER_US
    floor_us = ctas * tiles * tile_bytes / HBM_BYTES_PER_US
    many = tiles >= MANY_SLICES_FROM_TILES and ctas * 8 < slots
    best, best_cost = 1, None
    for s in range(1, (MAX_SPLITS_MANY if many else MAX_SPLITS) + 1):
        cap = cluster_capacity[s] if cluster_capacity and s < len(cluster_capacity) else 0
        if cap > 0:
            rounds, fixed = -(-ctas // cap), CLUSTER_OVERHEAD_US
            if rounds == 1 and ctas > cap * CLUSTER_FILL:
                rounds = 2
        else:
            rounds, fixed = -(-ctas * s // slots), SPLIT_OVERHEAD_US
        cost = max(floor_us, rounds * -(-tiles // s) * tile_us) + fixed + PER_SLICE_US * s + WAVE_PENALTY_US * (rounds - 1)
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


def decode_splits(n_dec: int, ctas_per_split: int, num_sms: int, cluster_capacity=None, tiles: int = 32,
                  tile_bytes: int = 32768) -> int:
    """Slices of the context per decoded token: the count with the least estimated time
    max(bytes / bandwidth, rounds x tiles per slice x time of a tile) + overheads, for contexts
    of ``tiles`` tiles of ``tile_bytes`` bytes (keys and values of one kv head).
    cluster_capacity[s], where given and not 0, is how many clusters of s slices the device
    holds at once: the decode kernel merges such slices itself (csrc/attention_mma.cu)."""
    cap = tuple(cluster_capacity) if cluster_capacity else None
    return _decode_splits(n_dec, ctas_per_split, num_sms, cap, int(tiles), int(tile_bytes), FORCED_SPLITS)


class Attention:
    """params: hidden_size, num_heads, num_kv_heads, head_dim, window (None = all
    keys), position (PartSpec)."""

    def __init__(self, spec, ctx):
        self.ctx = ctx
        self.hidden = int(spec["hidden_size"])
        self.nh = int(spec["num_heads"])
        self.nkv = int(spec["num_kv_heads"])
        self.d = int(spec["head_dim"])
        self.window = spec.get("window") or None
        if self.nh % self.nkv:
            raise ValueError(f"{self.nh} heads are not a multiple of {self.nkv} kv heads")
        if self.d > 256:
            raise ValueError(f"head size {self.d} is beyond what the attention kernels take (256)")
        self.position = build_position(spec["position"], ctx)
        self.scale = 1.0 / math.sqrt(self.d)
        self.qkv_width = (self.nh + 2 * self.nkv) * self.d
        self.num_sms = torch.cuda.get_device_properties(ctx.device).multi_processor_count \
            if ctx.device.type == "cuda" else 148
        ws, T = ctx.workspace, ctx.max_tokens
        ws.reserve("qkv", T * self.qkv_width, ctx.act_dtype)
        ws.reserve("attn_out", T * self.nh * self.d, ctx.act_dtype)
        ws.reserve("mixer_out", T * self.hidden, ctx.act_dtype)
        gchunks = -(-(self.nh // self.nkv) // 16)
        self._ctas_per_split = self.nkv * gchunks
        self._cluster_cap = None
        if ctx.device.type == "cuda":
            self._cluster_cap = [0] + [ops.attn_decode_cluster_capacity(ctx.act_dtype, self.d, s, self.nh // self.nkv)
                                       for s in range(1, ops.ATTN_MAX_CLUSTER + 1)]
        esize = torch.empty((), dtype=ctx.act_dtype).element_size()
        self._tile_bytes = TILE_KEYS * self.d * 2 * esize          # keys and values of one kv head
        rows = max(n * self._splits(n, TILE_KEYS << b) for n in range(1, ctx.max_seqs + 1)
                   for b in range(MAX_TILES.bit_length()))
        ws.reserve("attn_part_o", rows * self.nh * self.d, torch.float32)
        ws.reserve("attn_part_ml", rows * self.nh * 2, torch.float32)
        self._flat_ok = (ctx.device.type == "cuda" and ctx.act_dtype == torch.bfloat16 and self.d in (64, 128)
                         and ATTN_POLICY != "general" and FLAT_DECODE_FILL > 0
                         and ctx.max_seqs <= ops.ATTN_FLAT_MAX_SEQS)
        if self._flat_ok:
            pieces = ops.attn_decode_flat_pieces(ctx.max_seqs, self.nh, self.nkv, self.d)
            ws.reserve("attn_part_o", pieces * 16 * self.d, torch.float32)
            ws.reserve("attn_part_ml", pieces * 16 * 2, torch.float32)
            ws.reserve("attn_flat_prefix", ops.attn_decode_flat_prefix_ints(ctx.max_seqs, self.nh, self.nkv), torch.int32)
        self.w_qkv = None
        self.w_o = None

    def cache_need(self):
        return PagedKVNeed(self.nkv, self.d, self.window)

    def query_tiles(self):
        """The tile lists of the prompt kernels this mixer can end up using."""
        need = [TILES_GENERAL]
        if self.ctx.act_dtype == torch.bfloat16 and self.d in (64, 128) and ATTN_POLICY != "general":
            need.append(TILES_MMA)
            if ATTN_POLICY == "auto":
                need.append(TILES_TC)
        return need

    def _splits(self, n_dec: int, max_context: int) -> int:
        return decode_splits(n_dec, self._ctas_per_split, self.num_sms, self._cluster_cap,
                             context_tiles(max_context, self.window), self._tile_bytes)

    def _few_short_tiles(self, tiles128: int, batch) -> bool:
        """Prompt portions that leave the tcgen05 kernel's tiles (128 rows of two heads) on fewer
        than half of the SMs, with at most 256 keys each: the mma.sync kernel's tiles of 64 rows
        of one head spread the same work over four times the CTAs and start faster.  Measured on
        whole prompt steps of the Llama-3.1-8B shape (ms, tcgen05 / mma.sync): 64 tokens 4.10 /
        3.84, 128 tokens 4.45 / 4.24, 256 tokens 5.2-5.6 / 5.3-5.4, 512 tokens 8.3-8.5 / 8.6."""
        if tiles128 * ((self.nh + 1) // 2) * 2 > self.num_sms:
            return False
        return max(s + n for s, n in zip(batch.q_starts, batch.q_lens) if n > 1) <= SHORT_PROMPT_KEYS

    def _flat_step(self, n_dec: int) -> bool:
        """More (token, kv head) pairs than CTAs fit at once: equal ranges of tiles, no slices."""
        return bool(self._flat_ok and n_dec * self._ctas_per_split >= FLAT_DECODE_FILL * CTAS_PER_SM * self.num_sms)

    def step_tags(self, facts):
        """The count of slices this step's decoded tokens would be cut into: a step that is
        captured with one count is replayed only for steps that choose the same."""
        n = facts.num_seqs if facts.decode_only else 0
        if n == 0 or self._flat_step(n):
            return ()
        return (f"kv_slices={self._splits(n, facts.max_context)}",)

    def weights(self):
        return {"q_proj.weight": WeightSpec((self.nh * self.d, self.hidden)),
                "k_proj.weight": WeightSpec((self.nkv * self.d, self.hidden)),
                "v_proj.weight": WeightSpec((self.nkv * self.d, self.hidden)),
                "o_proj.weight": WeightSpec((self.hidden, self.nh * self.d))}

    def load(self, get):
        q, k, v = get("q_proj.weight"), get("k_proj.weight"), get("v_proj.weight")
        dt = torch.float32 if torch.float32 in (q.dtype, k.dtype, v.dtype) else q.dtype
        self.w_qkv = torch.cat([q.to(dt), k.to(dt), v.to(dt)], dim=0).contiguous()
        self.w_o = get("o_proj.weight").contiguous()

    # the optional protocol of parts/linear.py
    def takes_normed_rows(self, num_tokens):
        return fuses_norms(num_tokens, self.w_qkv, self.ctx.act_dtype)

    def fuses_next_norm(self, num_tokens):
        return fuses_norms(num_tokens, self.w_o, self.ctx.act_dtype)

    def _decode(self, qkv, kc, vc, group, batch, out, window, flat_step, fused, table, writes_cache):
        """The step's single decoded tokens (batch.dec_seqs) against the cache."""
        ws, n, bt = self.ctx.workspace, batch.num_decode, batch.block_tables[group]
        if flat_step:
            # more pairs than CTAs at once: equal ranges of tiles instead of whole slices
            pieces = ops.attn_decode_flat_pieces(n, self.nh, self.nkv, self.d)
            ops.attn_decode_flat(qkv, self.qkv_width, kc, vc, bt, batch.bt_stride, batch.cu_q_lens,
                                 batch.context_lens, batch.dec_seqs, n,
                                 ws.get("attn_part_o", 1, pieces * 16 * self.d),
                                 ws.get("attn_part_ml", 1, pieces * 16 * 2),
                                 ws.get("attn_flat_prefix", 1, ops.attn_decode_flat_prefix_ints(n, self.nh, self.nkv)), out,
                                 self.nh, self.nkv, self.d,
                                 self.ctx.page_size, window, self.scale)
            return
        facts = getattr(batch, "facts", None)
        longest = facts.max_context if facts is not None else max(s + q for s, q in zip(batch.q_starts, batch.q_lens))
        splits = self._splits(n, longest)
        part_o = ws.get("attn_part_o", 1, n * self.nh * splits * self.d)
        part_ml = ws.get("attn_part_ml", 1, n * self.nh * splits * 2)
        if fused:
            ops.attn_decode_rope(qkv, kc, vc, bt, batch.bt_stride, batch.cu_q_lens, batch.context_lens,
                                 batch.dec_seqs, n, splits, part_o, part_ml, out, self.nh,
                                 self.nkv, self.d, self.ctx.page_size, window, self.scale, batch.positions,
                                 batch.slot_mapping[group], table, writes_cache)
        else:
            ops.attn_decode(qkv, self.qkv_width, kc, vc, bt, batch.bt_stride, batch.cu_q_lens,
                            batch.context_lens, batch.dec_seqs, n, splits,
                            part_o, part_ml, out, self.nh, self.nkv, self.d, self.ctx.page_size, window, self.scale)

    def forward(self, x, batch, cache, writes_cache=True, then=None):
        T = x.shape[0]
        ws = self.ctx.workspace
        kc, vc, group = cache
        qkv = ws.get("qkv", T, self.qkv_width)
        linear(x, self.w_qkv, qkv)
        if hasattr(self.position, "apply"):
            # a position encoding that is not a rotation table: it rewrites q and k itself
            self.position.apply(qkv, batch, self.nh, self.nkv, self.d)
        # a step of decoded tokens only: the decode kernel rotates and writes the cache itself
        table = self.position.rope_table()
        flat_step = self._flat_step(batch.num_decode)
        fused = (FUSE_DECODE_ROPE and batch.num_decode > 0 and not batch.num_portions and ATTN_POLICY != "general"
                 and not flat_step
                 and not hasattr(self.position, "apply")
                 and ops.attn_decode_rope_ok(qkv.dtype, self.nh, self.nkv, self.d, table, self.position.interleaved))
        if not fused:
            ops.rope_kv_write(qkv, batch.positions, batch.slot_mapping[group], table,
                              kc, vc, self.nh, self.nkv, self.d, self.ctx.page_size,
                              self.position.interleaved, writes_cache)
        out = ws.get("attn_out", T, self.nh * self.d)
        window = int(self.window or 0)
        bt = batch.block_tables[group]
        if batch.num_portions:
            if TILES_GENERAL not in batch.tiles:
                raise RuntimeError("the step's batch was built without the index lists this mixer declares in "
                                   "query_tiles(): give them to the BatchBuilder (query_tiles=...)")
            t16, t64, t128 = batch.tiles[TILES_GENERAL], batch.tiles.get(TILES_MMA), batch.tiles.get(TILES_TC)
            if t128 is not None and t64 is not None and self._few_short_tiles(t128.count, batch):
                t128 = None
            ops.attn_prefill(qkv, self.qkv_width, kc, vc, bt, batch.bt_stride, batch.cu_q_lens,
                             batch.context_lens, t16.seq, t16.q0, t16.count,
                             out, self.nh, self.nkv, self.d, self.ctx.page_size, window, self.scale,
                             t64.seq if t64 else None, t64.q0 if t64 else None, t64.count if t64 else 0,
                             allow_mma=t64 is not None,
                             tile128_seq=t128.seq if t128 else None, tile128_q0=t128.q0 if t128 else None,
                             num_tiles128=t128.count if t128 else 0, allow_tc=t128 is not None)
        if batch.num_decode:
            self._decode(qkv, kc, vc, group, batch, out, window, flat_step, fused, table, writes_cache)
        y = ws.get("mixer_out", T, self.hidden)
        return linear(out, self.w_o, y, then)


register_mixer("attention", Attention)
