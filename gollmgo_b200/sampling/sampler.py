"""Token selection on the device from the step's float32 logits.

Greedy rows go through the arg-max kernel; as soon as one row of the step has a
temperature, the whole step goes through the sampling kernel (which still picks
greedily for rows with temperature 0).  Draw n of a request is a function of
(its seed, n) only, so its tokens do not depend on what else is in the batch
(the reference draws from one stream per engine: internal/engine/sampling.go:29-37).
"""
from __future__ import annotations

from typing import List, Sequence

import torch

from ..csrc import ops
from .params import SamplingParams

_MASK63 = (1 << 63) - 1


def _as_i64(x: int) -> int:
    """A 64-bit pattern as the signed value torch stores."""
    x &= (1 << 64) - 1
    return x - (1 << 64) if x >> 63 else x


class Sampler:
    """Samples on the device into ``tokens`` (a buffer the next step can read from
    directly) and copies the result to one of two pinned host buffers; ``wait``
    hands the tokens to the host.  Two steps can be in flight."""

    def __init__(self, device, max_rows: int, tokens: torch.Tensor = None):
        self.device = torch.device(device)
        self.max_rows = max_rows
        self.tokens = tokens if tokens is not None else torch.empty(max_rows, dtype=torch.int32, device=self.device)
        self._host = [torch.empty(max_rows, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._events = [torch.cuda.Event(), torch.cuda.Event()]
        self._turn = 0

    def sample_async(self, logits: torch.Tensor, params: Sequence[SamplingParams],
                     draw_index: Sequence[int]):
        """Launch the sampling of one token per row of ``logits`` [R, V]; ``draw_index[r]``
        is how many tokens request r has drawn before.  Returns a handle for ``wait``."""
        R = logits.shape[0]
        if R > self.max_rows:
            raise ValueError(f"{R} rows to sample, room for {self.max_rows}")
        slot = self._turn
        self._turn ^= 1
        if R == 0:
            return (slot, 0)
        out = self.tokens[:R]
        if all(p.greedy for p in params):
            ops.argmax(logits, out)
        else:
            dev = self.device
            temps = torch.tensor([p.temperature for p in params], dtype=torch.float32).to(dev, non_blocking=True)
            top_k = torch.tensor([p.top_k for p in params], dtype=torch.int32).to(dev, non_blocking=True)
            top_p = torch.tensor([p.top_p for p in params], dtype=torch.float32).to(dev, non_blocking=True)
            seeds = torch.tensor([_as_i64(p.seed or 0) for p in params], dtype=torch.int64).to(dev, non_blocking=True)
            draws = torch.tensor(list(draw_index), dtype=torch.int64).to(dev, non_blocking=True)
            ops.sample(logits, temps, top_k, top_p, seeds, draws, out)
        self._host[slot][:R].copy_(out, non_blocking=True)
        self._events[slot].record()
        return (slot, R)

    def wait(self, handle) -> List[int]:
        slot, R = handle
        if R == 0:
            return []
        self._events[slot].synchronize()
        return self._host[slot][:R].tolist()

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               draw_index: Sequence[int]) -> List[int]:
        return self.wait(self.sample_async(logits, params, draw_index))
