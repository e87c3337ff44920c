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
    def __init__(self, device, max_rows: int):
        self.device = torch.device(device)
        self.max_rows = max_rows
        self.out = torch.empty(max_rows, dtype=torch.int32, device=self.device)
        self.out_host = torch.empty(max_rows, dtype=torch.int32, pin_memory=True)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               draw_index: Sequence[int]) -> List[int]:
        """One token per row of ``logits`` [R, V]; ``draw_index[r]`` is how many tokens
        request r has drawn before."""
        R = logits.shape[0]
        if R == 0:
            return []
        if R > self.max_rows:
            raise ValueError(f"{R} rows to sample, room for {self.max_rows}")
        out = self.out[:R]
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
        self.out_host[:R].copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self.out_host[:R].tolist()
