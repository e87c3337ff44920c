"""Engine options.  Names and defaults are the reference's server config keys
(internal/config/config.go:33-78): max_batch_size 64, max_token_budget 4096,
max_queue_depth 256, prefill_chunk_size 512, block_size 16, max_memory_fraction 0.9."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class EngineConfig:
    dtype: str = "bfloat16"                # "bfloat16" (serving kernels) | "float32" (true 32-bit)
    block_size: int = 16                   # tokens per cache page
    num_blocks: Optional[int] = None       # pages per cache group; None => from max_memory_fraction
    max_memory_fraction: float = 0.9
    max_batch_size: int = 64               # sequences per step
    max_token_budget: int = 4096           # tokens per step
    max_queue_depth: int = 256
    prefill_chunk_size: int = 512          # most prompt tokens of one request per step; 0 = no cut
    max_model_len: Optional[int] = None    # longest sequence; None => max_position_embeddings
    strict_fcfs: bool = True               # the head of the queue blocks those behind it; False: a
                                           # request that does not fit is passed over, as in the
                                           # reference (internal/scheduler/fcfs.go:130-161)
    cuda_graphs: bool = True               # capture decode-only steps
    capture_at_start: bool = True          # capture every batch bucket when the engine is built, not at first use
    device: int = 0

    def validate(self) -> None:
        if self.dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype must be bfloat16 or float32, got {self.dtype!r}")
        if self.block_size <= 0 or self.block_size & (self.block_size - 1):
            raise ValueError(f"block_size must be a power of two, got {self.block_size}")
        if self.max_batch_size <= 0:
            raise ValueError("max_batch_size must be positive")
        if self.max_token_budget <= 0:
            raise ValueError("max_token_budget must be positive")
        if not (0.0 < self.max_memory_fraction <= 1.0):
            raise ValueError("max_memory_fraction must be in (0, 1]")
        if self.prefill_chunk_size < 0:
            raise ValueError("prefill_chunk_size must be >= 0")
