"""Build-time context shared by the parts of one model: dtype, device, step
limits, and a workspace of named activation buffers that parts share.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch


@dataclass(frozen=True)
class QueryTiles:
    """An index list a mixer asks the batch builder for: the query rows of every prompt
    portion (a sequence with more than one token in the step) cut into tiles of ``height``
    rows, as (sequence, first row) pairs; ``most_keys_first`` orders them by how many keys
    they attend to, longest first.  A mixer names the lists it wants in ``query_tiles()``;
    the step's batch then holds each under ``batch.tiles[that QueryTiles]``."""
    height: int
    most_keys_first: bool = False


@dataclass(frozen=True)
class StepFacts:
    """What is known of a step before its batch is built; parts may derive step tags from it
    (``step_tags(facts)``): steps with different tags are steps of different kinds, each with
    captured graphs of its own, and ``batch.tags`` tells a part which kind it is in."""
    num_seqs: int
    num_tokens: int
    decode_only: bool
    max_context: int              # most tokens any live request holds in the cache


class Workspace:
    """Named buffers, one allocation per name sized for the largest request.
    Parts ask for a buffer by name at build time and take a view of its first
    rows each step; two parts that use the same name share the memory, so a
    name must not be live across a call into another part that uses it."""

    def __init__(self, device):
        self.device = device
        self._want: Dict[str, Tuple[int, torch.dtype]] = {}
        self._bufs: Dict[str, torch.Tensor] = {}
        self._views: Dict[Tuple[str, int, int], torch.Tensor] = {}

    def reserve(self, name: str, numel: int, dtype: torch.dtype) -> None:
        old = self._want.get(name)
        if old is not None and old[1] != dtype:
            raise ValueError(f"workspace buffer {name!r} wanted as {old[1]} and {dtype}")
        self._want[name] = (max(numel, old[0] if old else 0), dtype)
        if name in self._bufs and self._bufs[name].numel() < self._want[name][0]:
            del self._bufs[name]
            self._views = {k: v for k, v in self._views.items() if k[0] != name}

    def get(self, name: str, rows: int, cols: int) -> torch.Tensor:
        """View [rows, cols] of the named buffer (views are kept: a step asks for the same few
        again and again, and making one costs microseconds of host time)."""
        key = (name, rows, cols)
        view = self._views.get(key)
        if view is not None:
            return view
        buf = self._bufs.get(name)
        if buf is None:
            numel, dtype = self._want[name]
            buf = torch.empty(numel, dtype=dtype, device=self.device)
            self._bufs[name] = buf
        n = rows * cols
        if n > buf.numel():
            raise ValueError(f"workspace buffer {name!r} holds {buf.numel()} elements, {n} asked")
        view = buf[:n].view(rows, cols)
        if len(self._views) > 4096:
            self._views.clear()
        self._views[key] = view
        return view

    def nbytes(self) -> int:
        return sum(n * torch.empty((), dtype=dt).element_size() for n, dt in self._want.values())


class BuildContext:
    def __init__(self, act_dtype: torch.dtype, device, max_tokens: int, max_seqs: int,
                 page_size: int, workspace: Optional[Workspace] = None):
        self.act_dtype = act_dtype
        self.device = torch.device(device)
        self.max_tokens = max_tokens          # most tokens in one step
        self.max_seqs = max_seqs              # most sequences in one step
        self.page_size = page_size
        self.workspace = workspace or Workspace(self.device)
