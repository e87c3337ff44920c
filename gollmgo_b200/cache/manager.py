"""The cache manager: keys and values in pages, a block table per request and
group, and state slots.

Layers are grouped by what they need of the cache.  A *paged* need is
(kv heads, head size, window); layers with equal needs share one group: one page
pool, one block table per request, one device tensor of shape
``[layers of the group, 2 (k, v), pages, kv heads, page size, head size]``, so
one page id addresses every layer of the group.  A group with a window gives a
page back as soon as every token in it is behind the window of all future
queries.  A *fixed-state* need is a tensor shape per request; its buffer is
indexed by the request's state slot.

Reference: internal/kvcache/block_pool.go, block_table.go (one group, no window,
no state), kernels/gollmgo_kvcache.cu:11-63 (device layout [layer][slot][head][d]).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .pool import OutOfPages, PagePool
from .state_slots import StateSlots


@dataclass(frozen=True)
class PagedKVNeed:
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None      # None: all keys are kept


@dataclass(frozen=True)
class FixedStateNeed:
    shape: Tuple[int, ...]            # per request
    dtype: str = "float32"


@dataclass
class PagedGroup:
    need: PagedKVNeed
    cache_ids: List[int]              # which cache entries (run-order caches) live here
    pool: PagePool
    kv: object = None                 # device tensor [n, 2, pages, nkv, page, d] or None on the host


@dataclass
class RequestCache:
    state_slot: int
    num_tokens: int = 0
    pages: List[List[int]] = field(default_factory=list)   # per group: logical page -> id, -1 = given back


@dataclass(frozen=True)
class Appended:
    start: int                         # tokens cached before
    slots: List[np.ndarray]            # per group: flat slot (page * page_size + offset) per new token, int32


class CacheManager:
    def __init__(self, needs: Sequence[object], page_size: int, num_pages: int,
                 max_requests: int, dtype=None, device=None):
        if page_size <= 0 or page_size & (page_size - 1):
            raise ValueError(f"page size must be a power of two, got {page_size}")
        self.page_size = page_size
        self.num_pages = num_pages
        self.groups: List[PagedGroup] = []
        self.group_of: Dict[int, Tuple[int, int]] = {}        # cache id -> (group, index in group)
        self.state_needs: Dict[int, FixedStateNeed] = {}
        self.state_buffers: Dict[int, object] = {}
        self.slots = StateSlots(max_requests)
        self.requests: Dict[object, RequestCache] = {}
        # flat mirrors for the native step packer (csrc/host_pack.cu): per group a table
        # [state slot, logical page] of page ids (-1 = none), and the tokens cached per slot
        self.max_requests = max_requests
        self.poison_freed = os.environ.get("GOLLMGO_B200_POISON_FREED", "0") == "1"
        self.tab: List[np.ndarray] = []
        self.ntok = np.zeros(max_requests, dtype=np.int32)
        for cid, need in enumerate(needs):
            if need is None:
                continue
            if isinstance(need, PagedKVNeed):
                for gi, g in enumerate(self.groups):
                    if g.need == need:
                        self.group_of[cid] = (gi, len(g.cache_ids))
                        g.cache_ids.append(cid)
                        break
                else:
                    self.group_of[cid] = (len(self.groups), 0)
                    self.groups.append(PagedGroup(need, [cid], PagePool(num_pages)))
            elif isinstance(need, FixedStateNeed):
                self.state_needs[cid] = need
            else:
                raise TypeError(f"cache need of entry {cid} is {type(need).__name__}")
        self.tab = [np.full((max_requests, 64), -1, dtype=np.int32) for _ in self.groups]
        self.any_window = any(g.need.window is not None for g in self.groups)
        if device is not None:
            import torch
            for g in self.groups:
                g.kv = torch.zeros(len(g.cache_ids), 2, num_pages, g.need.n_kv_heads, page_size,
                                   g.need.head_dim, dtype=dtype, device=device)
            for cid, need in self.state_needs.items():
                self.state_buffers[cid] = torch.zeros(max_requests, *need.shape,
                                                      dtype=getattr(torch, need.dtype), device=device)

    # ------------------------------------------------------------------ sizes
    @staticmethod
    def bytes_per_page(needs: Sequence[object], page_size: int, element_size: int) -> int:
        """Bytes one page id costs over all groups (each group has its own pool of
        ``num_pages``, so this is the cost of adding one page to every pool)."""
        total = 0
        for need in needs:
            if isinstance(need, PagedKVNeed):
                total += 2 * need.n_kv_heads * need.head_dim * page_size * element_size
        return total

    def layer_cache(self, cache_id: int):
        """(k, v) tensors [pages, nkv, page, d] of one cache entry, and its group index."""
        gi, idx = self.group_of[cache_id]
        g = self.groups[gi]
        return g.kv[idx, 0], g.kv[idx, 1], gi

    def _give_back(self, gi: int, page: int) -> None:
        """Return a page of group gi to its pool.  With GOLLMGO_B200_POISON_FREED=1 its keys and
        values are overwritten with NaN on the device first (in stream order, so after every
        step launched so far): a kernel that read a page its request no longer holds would
        then show up as NaN logits."""
        g = self.groups[gi]
        if self.poison_freed and g.kv is not None:
            g.kv[:, :, page] = float("nan")
        g.pool.release(page)

    # ------------------------------------------------------------------ requests
    def admit(self, req_id) -> int:
        if req_id in self.requests:
            raise RuntimeError(f"request {req_id!r} is already admitted")
        slot = self.slots.take()
        self.requests[req_id] = RequestCache(slot, 0, [[] for _ in self.groups])
        for t in self.tab:
            t[slot, :] = -1
        self.ntok[slot] = 0
        for buf in self.state_buffers.values():
            buf[slot].zero_()
        return slot

    def num_tokens(self, req_id) -> int:
        return self.requests[req_id].num_tokens

    def _behind_window(self, rc: RequestCache, gi: int) -> List[int]:
        """Logical pages of group gi that no future query of the request can see."""
        w = self.groups[gi].need.window
        if w is None:
            return []
        first_needed = rc.num_tokens - w + 1          # oldest key the next token may read
        out = []
        for idx, page in enumerate(rc.pages[gi]):
            if (idx + 1) * self.page_size > first_needed:
                break
            if page >= 0:
                out.append(idx)
        return out

    def pages_short(self, req_id, n_tokens: int) -> int:
        """How many pages are lacking (max over groups) to append n_tokens; 0 = it fits."""
        rc = self.requests[req_id]
        short = 0
        for gi, g in enumerate(self.groups):
            have = len(rc.pages[gi])
            want = -(-(rc.num_tokens + n_tokens) // self.page_size)
            free = g.pool.num_free + len(self._behind_window(rc, gi))
            short = max(short, (want - have) - free)
        return max(short, 0)

    def pages_delta(self, req_id, n_tokens: int) -> List[Tuple[int, int]]:
        """Per group (taken, given back): the pages that appending the next n_tokens of the
        request takes from the group's pool, and the pages behind a window that go back to it
        first.  ``append`` succeeds iff taken <= free + given back in every group.  A request
        that is not admitted (or ``None``) holds nothing yet.  This is what a scheduler plans
        with: it never redoes the page arithmetic of a group itself."""
        rc = self.requests.get(req_id) if req_id is not None else None
        out = []
        for gi in range(len(self.groups)):
            have = len(rc.pages[gi]) if rc else 0
            held = rc.num_tokens if rc else 0
            want = -(-(held + n_tokens) // self.page_size)
            out.append((max(want - have, 0), len(self._behind_window(rc, gi)) if rc else 0))
        return out

    def pages_held(self, req_id) -> List[int]:
        """Per group, how many pages the request holds now (what freeing it gives back)."""
        rc = self.requests.get(req_id)
        if rc is None:
            return [0] * len(self.groups)
        return [sum(1 for p in pages if p >= 0) for pages in rc.pages]

    def free_pages_per_group(self) -> List[int]:
        return [g.pool.num_free for g in self.groups]

    def capacity_tokens(self, portion: int = 1) -> Optional[int]:
        """Most tokens one request can ever hold: the pool of the smallest group that keeps
        every key.  A group with a window only has to hold the window and one step's portion
        (its older pages go back as the request grows); None = no group sets a limit (every
        group has a window that fits, or the model keeps no pages at all)."""
        limit = None
        for g in self.groups:
            pool = g.pool.num_pages * self.page_size
            if g.need.window is not None and pool >= g.need.window + portion + 2 * self.page_size:
                continue
            limit = pool if limit is None else min(limit, pool)
        return limit

    def append(self, req_id, n_tokens: int) -> Appended:
        """Make room for the next n_tokens of the request in every group, all or
        nothing; returns where they go.  Pages behind a window are given back first."""
        if n_tokens <= 0:
            raise ValueError("append needs at least one token")
        rc = self.requests[req_id]
        if self.pages_short(req_id, n_tokens):
            raise OutOfPages(f"request {req_id!r} needs {self.pages_short(req_id, n_tokens)} more "
                             f"pages than are free")
        start = rc.num_tokens
        ps = self.page_size
        slots = []
        for gi, g in enumerate(self.groups):
            for idx in self._behind_window(rc, gi):
                self._give_back(gi, rc.pages[gi][idx])
                rc.pages[gi][idx] = -1
            want = -(-(start + n_tokens) // ps)
            have = len(rc.pages[gi])
            rc.pages[gi].extend(g.pool.allocate(want - have))
            self._mirror(gi, rc, since=have if not self.any_window else 0)
            pos = np.arange(start, start + n_tokens, dtype=np.int32)
            slots.append(self.tab[gi][rc.state_slot, pos // ps] * ps + pos % ps)
        rc.num_tokens = start + n_tokens
        self.ntok[rc.state_slot] = rc.num_tokens
        return Appended(start, slots)

    def _mirror(self, gi: int, rc: RequestCache, since: int = 0) -> None:
        """Bring the flat table of group gi up to date with the request's pages (``since``: the
        entries before it are known to be unchanged)."""
        pages = rc.pages[gi]
        t = self.tab[gi]
        if len(pages) > t.shape[1]:
            wider = np.full((self.max_requests, max(2 * t.shape[1], len(pages))), -1, dtype=np.int32)
            wider[:, :t.shape[1]] = t
            self.tab[gi] = t = wider
        row = t[rc.state_slot]
        if since < len(pages):
            row[since:len(pages)] = pages[since:]
        row[len(pages):] = -1

    def append_one(self, req_id) -> int:
        """append(req_id, 1) for the step packer: returns the position of the new token.  Where
        the token lands in a page the request already holds (and no group has a window to
        slide), nothing but the count changes."""
        rc = self.requests[req_id]
        start = rc.num_tokens
        if self.any_window or start % self.page_size == 0:
            return self.append(req_id, 1).start
        rc.num_tokens = start + 1
        self.ntok[rc.state_slot] = start + 1
        return start

    def rollback(self, req_id, num_tokens: int) -> None:
        """Forget the tokens after the first ``num_tokens`` and give back the pages
        that held only those (used when a step is abandoned while it is built)."""
        rc = self.requests[req_id]
        if num_tokens > rc.num_tokens or num_tokens < 0:
            raise ValueError("rollback beyond what the request holds")
        keep = -(-num_tokens // self.page_size)
        for gi, g in enumerate(self.groups):
            while len(rc.pages[gi]) > keep:
                page = rc.pages[gi].pop()
                if page >= 0:
                    self._give_back(gi, page)
            self._mirror(gi, rc)
        rc.num_tokens = num_tokens
        self.ntok[rc.state_slot] = num_tokens

    def block_table(self, req_id, group: int) -> List[int]:
        return self.requests[req_id].pages[group]

    def state_slot(self, req_id) -> int:
        return self.requests[req_id].state_slot

    def free(self, req_id) -> None:
        """Give back everything the request holds."""
        rc = self.requests.pop(req_id)
        for gi, g in enumerate(self.groups):
            for page in rc.pages[gi]:
                if page >= 0:
                    self._give_back(gi, page)
        for t in self.tab:
            t[rc.state_slot, :] = -1
        self.ntok[rc.state_slot] = 0
        self.slots.give_back(rc.state_slot)

    # ------------------------------------------------------------------ checks
    def free_pages(self, group: int = 0) -> int:
        return self.groups[group].pool.num_free

    def min_free_pages(self) -> int:
        return min((g.pool.num_free for g in self.groups), default=self.num_pages)

    def audit(self) -> None:
        """Raise if a page is lost, held twice, or both free and held."""
        for gi, g in enumerate(self.groups):
            held: Dict[int, object] = {}
            for rid, rc in self.requests.items():
                for page in rc.pages[gi]:
                    if page < 0:
                        continue
                    if page in held:
                        raise AssertionError(f"group {gi}: page {page} held by {held[page]!r} and {rid!r}")
                    held[page] = rid
            free = g.pool.free_pages()
            if len(set(free)) != len(free):
                raise AssertionError(f"group {gi}: a page is on the free list twice")
            both = set(free) & set(held)
            if both:
                raise AssertionError(f"group {gi}: pages {sorted(both)} are free and held")
            if len(free) + len(held) != g.pool.num_pages:
                raise AssertionError(f"group {gi}: {g.pool.num_pages - len(free) - len(held)} pages lost")
            for page in held:
                if g.pool.refcount(page) != 1:
                    raise AssertionError(f"group {gi}: page {page} has count {g.pool.refcount(page)}")
        slots = [rc.state_slot for rc in self.requests.values()]
        if len(set(slots)) != len(slots) or sorted(slots) != self.slots.held():
            raise AssertionError("state slots and requests disagree")
        # the flat mirrors say the same as the requests, and nothing for slots nobody holds
        for gi in range(len(self.groups)):
            want = np.full_like(self.tab[gi], -1)
            for rc in self.requests.values():
                want[rc.state_slot, :len(rc.pages[gi])] = rc.pages[gi]
            if not np.array_equal(want, self.tab[gi]):
                raise AssertionError(f"group {gi}: the flat page table disagrees with the requests")
        counts = np.zeros_like(self.ntok)
        for rc in self.requests.values():
            counts[rc.state_slot] = rc.num_tokens
        if not np.array_equal(counts, self.ntok):
            raise AssertionError("the flat token counts disagree with the requests")
