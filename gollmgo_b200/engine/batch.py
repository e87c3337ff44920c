"""One step's batch: flat token arrays plus per-sequence metadata, built on the
host and sent to the device in one copy.

The reference's Batch (internal/backend/runner.go:30-53) carries a per-token slot
list for every sequence, rebuilt each step, and its CUDA bridge splits a mixed
batch into a prompt call and a decode call (internal/backend/cuda/model_bridge.go:305-383).
Here a batch is any mix of portions (one token or many) and runs as one forward
pass; the device gets block tables, not per-token slot lists.

The builder knows nothing of any kernel.  Index lists over the query rows of prompt
portions are built only as the model's mixers ask for them (``QueryTiles``: a tile
height and an order); a model whose mixers ask for none gets none.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..parts.context import QueryTiles


@dataclass
class StepEntry:
    """The next tokens of one request and the places among them whose logits are wanted."""
    request_id: object
    tokens: Sequence[int]
    want: Sequence[int] = ()
    # the entry's single token is not known on the host yet: it is row `token_src` of the
    # tokens sampled on the device in the step before (tokens[0] is then ignored)
    token_src: int = -1
    # the caller has checked that every token id is inside the vocabulary (the engine does when a
    # request is added): the step function does not go over them again
    checked: bool = False


class TileList:
    """One QueryTiles list of a step on the device: tile i covers rows q0[i] .. q0[i] + height
    of sequence seq[i] (``count`` tiles)."""

    def __init__(self, need: QueryTiles, seq: torch.Tensor, q0: torch.Tensor, count: int):
        self.need, self.seq, self.q0, self.count = need, seq, q0, count


class StepBatch:
    """Device views (int32 unless noted) and host facts of one step."""
    num_tokens: int
    num_seqs: int
    num_logit_rows: int
    num_portions: int                      # sequences that bring more than one token (prompt portions)
    num_decode: int
    bt_stride: int
    token_ids: torch.Tensor
    token_src: Optional[torch.Tensor]      # None: every token id is given by the host
    prev_tokens: Optional[torch.Tensor]    # the tokens sampled on the device in the step before
    positions: torch.Tensor
    cu_q_lens: torch.Tensor
    context_lens: torch.Tensor
    state_slots: torch.Tensor
    logit_rows: torch.Tensor
    tiles: "dict[QueryTiles, TileList]"    # the index lists the model's mixers asked for
    dec_seqs: torch.Tensor
    tags: tuple = ()                       # the step's kind, as the model's parts tagged it (set by the runner)
    facts: object = None                   # the StepFacts the tags were made from (set by the runner)
    slot_mapping: List[torch.Tensor]
    block_tables: List[torch.Tensor]
    # host side
    request_ids: List[object]
    q_lens: List[int]
    q_starts: List[int]
    state_slot_list: List[int]


def _align(n: int) -> int:
    return (n + 3) & ~3


class BatchLayout:
    """Offsets of every array in the packed int32 buffer, for given capacities."""

    def __init__(self, T: int, B: int, R: int, tile_counts: Sequence[int], ND: int, G: int, stride: int):
        self.T, self.B, self.R, self.ND, self.G, self.stride = T, B, R, ND, G, stride
        self.tile_counts = list(tile_counts)
        off = 0

        def take(n):
            nonlocal off
            o = off
            off += _align(max(n, 1))
            return o
        self.token_ids = take(T)
        self.token_src = take(T)
        self.positions = take(T)
        self.slot_mapping = [take(T) for _ in range(G)]
        self.cu_q_lens = take(B + 1)
        self.context_lens = take(B)
        self.state_slots = take(B)
        self.logit_rows = take(R)
        self.tile_seq = [take(n) for n in self.tile_counts]
        self.tile_q0 = [take(n) for n in self.tile_counts]
        self.dec_seqs = take(ND)
        self.block_tables = [take(B * stride) for _ in range(G)]
        self.size = off


class BatchBuilder:
    """Turns step entries into a StepBatch, reserving cache room on the way.

    ``fixed_seqs`` and ``fixed_stride`` pin the layout (a captured decode step
    replays with the same addresses): sequences are padded to ``fixed_seqs`` with
    empty ones that no kernel touches.
    """

    def __init__(self, cache, device, capacity_ints: int = 1 << 16, query_tiles: Sequence[QueryTiles] = ()):
        self.cache = cache
        self.device = torch.device(device)
        self.G = len(cache.groups)
        self.query_tiles = list(dict.fromkeys(query_tiles))      # what the model's mixers asked for
        self._host = None
        self._dev = None
        self._copied = None
        # steps of single decoded tokens are packed by native code (GOLLMGO_B200_NATIVE_PACK=0: by the general path)
        self.native_decode = os.environ.get("GOLLMGO_B200_NATIVE_PACK", "1") != "0"
        self._ensure(capacity_ints)

    def decode_layout(self, seqs: int, stride: int) -> BatchLayout:
        """The layout of a step of ``seqs`` single tokens (what a captured step's buffer holds)."""
        return BatchLayout(seqs, seqs, seqs, [0] * len(self.query_tiles), seqs, self.G, stride)

    def _ensure(self, n: int) -> None:
        if self._host is not None and self._host.numel() >= n:
            return
        n = max(n, 1 << 12)
        cuda = self.device.type == "cuda"
        self._host = torch.empty(n, dtype=torch.int32, pin_memory=cuda)
        self._dev = torch.empty(n, dtype=torch.int32, device=self.device)
        self._copied = None

    def _build_decode(self, entries, fixed_seqs, fixed_stride, static_dev) -> StepBatch:
        """build() for a step in which every entry brings one token and wants its logits: the
        per-sequence arrays are packed by native code (csrc/host_pack.cu) from the cache
        manager's flat tables; the same layout and the same result as the general path."""
        cache = self.cache
        ids = [e.request_id for e in entries]
        B = len(ids)
        if len(set(ids)) != B:
            raise ValueError("a request appears twice in one step")
        Bp = fixed_seqs if fixed_seqs is not None else B
        if Bp < B:
            raise ValueError("more sequences than the fixed layout holds")
        starts: List[int] = []
        try:
            for rid in ids:
                starts.append(cache.append_one(rid))
            return self._pack_decode(entries, ids, starts, Bp, fixed_stride, static_dev)
        except Exception:
            # all or nothing: whatever fails from here on (no pages left, a layout that does not
            # fit, the native packer refusing its arguments) leaves the cache as it was
            for rid, s0 in zip(ids, starts):
                cache.rollback(rid, s0)
            raise

    def _pack_decode(self, entries, ids, starts, Bp, fixed_stride, static_dev) -> StepBatch:
        from ..csrc import ops
        cache, ps, G = self.cache, self.cache.page_size, self.G
        B = len(ids)
        reqs = cache.requests
        rcs = [reqs[rid] for rid in ids]
        slots = [rc.state_slot for rc in rcs]
        max_pages = max(len(p) for rc in rcs for p in rc.pages) if G else 1
        stride = fixed_stride if fixed_stride is not None else max(1, max_pages)
        if stride < max_pages:
            raise ValueError(f"a sequence holds {max_pages} pages, the fixed block table has {stride}")
        lay = self.decode_layout(Bp, stride)
        used = min(stride, max(1, max_pages))
        hlay = lay if used == stride else self.decode_layout(Bp, used)
        cuda = self.device.type == "cuda"
        if static_dev is None:
            self._ensure(lay.size)
            if self._copied is not None:
                self._copied.synchronize()
            host = self._host
        else:
            host = torch.empty(hlay.size, dtype=torch.int32, pin_memory=cuda)
        h = host.numpy()
        h[:hlay.size] = 0
        offsets = np.array([hlay.token_ids, hlay.token_src, hlay.positions, hlay.cu_q_lens, hlay.context_lens,
                            hlay.state_slots, hlay.logit_rows, hlay.dec_seqs, *hlay.slot_mapping,
                            *hlay.block_tables], dtype=np.int32)
        srcs = [e.token_src for e in entries]
        ops.pack_decode_step(h, offsets, G, B, Bp, used, ps,
                             np.array([e.tokens[0] for e in entries], dtype=np.int32),
                             np.array(srcs, dtype=np.int32), np.array(slots, dtype=np.int32),
                             np.array([s0 + 1 for s0 in starts], dtype=np.int32), cache.tab)
        dev = self._dev if static_dev is None else static_dev
        if dev.numel() < lay.size:
            raise ValueError("static batch buffer is too small for this layout")
        if hlay is lay:
            dev[:lay.size].copy_(host[:lay.size], non_blocking=cuda)
        else:
            head = lay.block_tables[0] if G else lay.size
            dev[:head].copy_(host[:head], non_blocking=cuda)
            for g in range(G):
                src = host[hlay.block_tables[g]:hlay.block_tables[g] + Bp * used].view(Bp, used)
                dev[lay.block_tables[g]:lay.block_tables[g] + Bp * stride].view(Bp, stride)[:, :used] \
                    .copy_(src, non_blocking=cuda)
        if cuda and static_dev is None:
            self._copied = torch.cuda.Event()
            self._copied.record()
        sb = StepBatch()
        sb.num_tokens, sb.num_seqs, sb.num_logit_rows = Bp, Bp, Bp
        sb.num_portions, sb.num_decode, sb.bt_stride = 0, Bp, stride
        v = lambda off, n: dev[off:off + max(n, 1)]
        sb.token_ids, sb.positions = v(lay.token_ids, Bp), v(lay.positions, Bp)
        sb.token_src = v(lay.token_src, Bp) if (static_dev is not None or any(x >= 0 for x in srcs)) else None
        sb.cu_q_lens, sb.context_lens = v(lay.cu_q_lens, Bp + 1), v(lay.context_lens, Bp)
        sb.state_slots, sb.logit_rows = v(lay.state_slots, Bp), v(lay.logit_rows, Bp)[:Bp]
        sb.tiles = {need: TileList(need, v(lay.tile_seq[i], 0), v(lay.tile_q0[i], 0), 0)
                    for i, need in enumerate(self.query_tiles)}
        sb.dec_seqs = v(lay.dec_seqs, Bp)
        sb.slot_mapping = [v(o, Bp) for o in lay.slot_mapping]
        sb.block_tables = [v(o, Bp * stride) for o in lay.block_tables]
        sb.request_ids, sb.q_lens, sb.q_starts = ids, [1] * B, starts
        sb.state_slot_list = slots
        sb.prev_tokens = None
        sb.layout = lay
        return sb

    def build(self, entries: Sequence[StepEntry], fixed_seqs: Optional[int] = None,
              fixed_stride: Optional[int] = None, static_dev: Optional[torch.Tensor] = None) -> StepBatch:
        cache, ps, G = self.cache, self.cache.page_size, self.G
        if not entries:
            raise ValueError("a step needs at least one entry")
        if self.native_decode and self.device.type == "cuda" and \
                all(len(e.tokens) == 1 and len(e.want) == 1 and e.want[0] == 0 for e in entries):
            return self._build_decode(entries, fixed_seqs, fixed_stride, static_dev)
        ids = [e.request_id for e in entries]
        if len(set(ids)) != len(ids):
            raise ValueError("a request appears twice in one step")
        # what can be checked without the cache is checked before it is touched
        for e in entries:
            if len(e.tokens) == 0:
                raise ValueError(f"request {e.request_id!r}: a step entry needs at least one token")
            for w in e.want:
                if not (0 <= w < len(e.tokens)):
                    raise ValueError(f"request {e.request_id!r}: wanted place {w} is outside its "
                                     f"{len(e.tokens)} tokens")
            if e.token_src >= 0 and len(e.tokens) != 1:
                raise ValueError("only a single decoded token can come from the device")
        if fixed_seqs is not None and fixed_seqs < len(entries):
            raise ValueError("more sequences than the fixed layout holds")
        appended = []
        try:
            for e in entries:
                appended.append(cache.append(e.request_id, len(e.tokens)))
            return self._pack(entries, ids, appended, fixed_seqs, fixed_stride, static_dev)
        except Exception:
            # all or nothing: whatever fails from here on (no pages left, a block table wider than
            # the fixed layout, a buffer that is too small) leaves the cache as it was; what was
            # appended in this call is rolled back by truncation
            for e, a in zip(entries, appended):
                cache.rollback(e.request_id, a.start)
            raise

    def _pack(self, entries, ids, appended, fixed_seqs, fixed_stride, static_dev) -> StepBatch:
        cache, ps, G = self.cache, self.cache.page_size, self.G
        B = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        q_starts = [a.start for a in appended]
        T = sum(q_lens)
        portions = [b for b in range(B) if q_lens[b] > 1]
        tile_lists = []
        for need in self.query_tiles:
            tl = [(b, q0) for b in portions for q0 in range(0, q_lens[b], need.height)]
            if need.most_keys_first:
                tl.sort(key=lambda t: -(q_starts[t[0]] + t[1]))
            tile_lists.append(tl)
        counts = [len(tl) for tl in tile_lists]
        dec = [b for b in range(B) if q_lens[b] == 1]
        max_pages = max(len(cache.block_table(e.request_id, g)) for e in entries for g in range(G)) if G else 1
        Bp = fixed_seqs if fixed_seqs is not None else B
        stride = fixed_stride if fixed_stride is not None else max(1, max_pages)
        if stride < max_pages:
            raise ValueError(f"a sequence holds {max_pages} pages, the fixed block table has {stride}")
        Tp = T + (Bp - B)            # padded sequences are given one dummy token each
        rows, base = [], 0
        for e, n in zip(entries, q_lens):
            rows.extend(base + w for w in e.want)
            base += n
        rows.extend(range(T, Tp))    # ... whose logits are computed and ignored
        R = len(rows)
        lay = BatchLayout(Tp, Bp, R, counts, len(dec) + (Bp - B), G, stride)
        # on the host the block tables are packed with only as many columns as are in use; with a
        # fixed (wide) device stride they are copied as a 2-d block, not as the whole table
        used = min(stride, max(1, max_pages))
        hlay = lay if used == stride else BatchLayout(Tp, Bp, R, counts, len(dec) + (Bp - B), G, used)
        if static_dev is None:
            self._ensure(lay.size)
            if self._copied is not None:
                self._copied.synchronize()
        host = self._host if static_dev is None else torch.empty(hlay.size, dtype=torch.int32,
                                                                  pin_memory=self.device.type == "cuda")
        h = host.numpy()
        h[:hlay.size] = 0
        h[lay.token_ids:lay.token_ids + T] = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
        h[lay.token_src:lay.token_src + Tp] = -1
        if any(e.token_src >= 0 for e in entries):
            base = 0
            for e, n in zip(entries, q_lens):
                if e.token_src >= 0:
                    h[lay.token_src + base] = e.token_src
                base += n
            has_src = True
        else:
            has_src = False
        pos = np.concatenate([np.arange(s, s + n, dtype=np.int32) for s, n in zip(q_starts, q_lens)])
        h[lay.positions:lay.positions + T] = pos
        for g in range(G):
            sm = h[lay.slot_mapping[g]:lay.slot_mapping[g] + Tp]
            sm[:] = -1
            sm[:T] = np.concatenate([a.slots[g] for a in appended])
        cu = np.zeros(Bp + 1, dtype=np.int32)
        cu[1:B + 1] = np.cumsum(q_lens)
        cu[B + 1:] = T + np.arange(1, Bp - B + 1)
        h[lay.cu_q_lens:lay.cu_q_lens + Bp + 1] = cu
        h[lay.context_lens:lay.context_lens + B] = [s + n for s, n in zip(q_starts, q_lens)]
        h[lay.state_slots:lay.state_slots + B] = [cache.state_slot(e.request_id) for e in entries]
        h[lay.state_slots + B:lay.state_slots + Bp] = -1
        h[lay.logit_rows:lay.logit_rows + R] = rows
        for i, tl in enumerate(tile_lists):
            if tl:
                h[lay.tile_seq[i]:lay.tile_seq[i] + len(tl)] = [t[0] for t in tl]
                h[lay.tile_q0[i]:lay.tile_q0[i] + len(tl)] = [t[1] for t in tl]
        nd = len(dec) + (Bp - B)
        h[lay.dec_seqs:lay.dec_seqs + len(dec)] = dec
        h[lay.dec_seqs + len(dec):lay.dec_seqs + nd] = -1
        for g in range(G):
            bt = h[hlay.block_tables[g]:hlay.block_tables[g] + Bp * used].reshape(Bp, used)
            bt[:] = -1
            for b, e in enumerate(entries):
                pages = cache.block_table(e.request_id, g)
                bt[b, :len(pages)] = pages
        dev = self._dev if static_dev is None else static_dev
        if dev.numel() < lay.size:
            raise ValueError("static batch buffer is too small for this layout")
        cuda = self.device.type == "cuda"
        if hlay is lay:
            dev[:lay.size].copy_(host[:lay.size], non_blocking=cuda)
        else:
            head = lay.block_tables[0] if G else lay.size          # everything before the block tables
            dev[:head].copy_(host[:head], non_blocking=cuda)
            for g in range(G):
                src = host[hlay.block_tables[g]:hlay.block_tables[g] + Bp * used].view(Bp, used)
                dev[lay.block_tables[g]:lay.block_tables[g] + Bp * stride].view(Bp, stride)[:, :used] \
                    .copy_(src, non_blocking=cuda)
        if cuda and static_dev is None:
            self._copied = torch.cuda.Event()
            self._copied.record()

        sb = StepBatch()
        sb.num_tokens, sb.num_seqs, sb.num_logit_rows = Tp, Bp, R
        sb.num_portions, sb.num_decode, sb.bt_stride = len(portions), nd, stride
        v = lambda off, n: dev[off:off + max(n, 1)]
        sb.token_ids, sb.positions = v(lay.token_ids, Tp), v(lay.positions, Tp)
        sb.token_src = v(lay.token_src, Tp) if (has_src or static_dev is not None) else None
        sb.cu_q_lens, sb.context_lens = v(lay.cu_q_lens, Bp + 1), v(lay.context_lens, Bp)
        sb.state_slots, sb.logit_rows = v(lay.state_slots, Bp), v(lay.logit_rows, R)[:R]
        sb.tiles = {need: TileList(need, v(lay.tile_seq[i], counts[i]), v(lay.tile_q0[i], counts[i]), counts[i])
                    for i, need in enumerate(self.query_tiles)}
        sb.dec_seqs = v(lay.dec_seqs, nd)
        sb.slot_mapping = [v(o, Tp) for o in lay.slot_mapping]
        sb.block_tables = [v(o, Bp * stride) for o in lay.block_tables]
        sb.request_ids, sb.q_lens, sb.q_starts = ids, q_lens, q_starts
        sb.state_slot_list = [cache.state_slot(e.request_id) for e in entries]
        sb.prev_tokens = None
        sb.layout = lay
        return sb
