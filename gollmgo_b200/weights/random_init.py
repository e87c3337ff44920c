"""Random weights: from a configuration and a seed, either straight onto a device
(benchmarks) or as a model folder with config.json and model.safetensors.

The value of a tensor depends only on (seed, tensor name, device kind), not on the
order in which tensors are made.  Matrices and tables are N(0, std); norm weights
are 1, or 1 + N(0, norm_jitter).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Callable, Dict

import torch

from .loader import WeightSpec
from .safetensors_io import save_file


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def random_tensor(name: str, spec: WeightSpec, seed: int, device, dtype: torch.dtype,
                  std: float = 0.02, norm_jitter: float = 0.0) -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed(_tensor_seed(seed, name))
    if len(spec.shape) == 1:                      # a norm's weight
        t = torch.ones(spec.shape, dtype=torch.float32, device=device)
        if norm_jitter:
            t += norm_jitter * torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device)
        return t.to(dtype)
    t = torch.empty(spec.shape, dtype=dtype, device=device)
    t.normal_(0.0, std, generator=gen)
    return t


def random_source(manifest: Dict[str, WeightSpec], seed: int, device, dtype: torch.dtype,
                  std: float = 0.02, norm_jitter: float = 0.0) -> Callable[[str], torch.Tensor]:
    """``get(name)`` that makes each tensor of the manifest on ``device``."""
    def get(name: str):
        spec = manifest[name]
        if spec.optional:                  # what the model can do without (the head of a tied model) is left out
            return None
        return random_tensor(name, spec, seed, device, dtype, std, norm_jitter)
    return get


def write_random_model(model_dir: str, config: dict, seed: int, dtype: str = "bfloat16",
                       std: float = 0.02, norm_jitter: float = 0.0, device="cpu") -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a config.json
    dict naming a registered architecture).  Returns ``model_dir``.  ``device``: where the
    numbers are drawn (a CUDA device draws a checkpoint of real layer sizes in seconds; the
    values depend on the kind of device, the file is the same kind of file)."""
    from ..parts.model import manifest_for_config      # late: parts imports weights
    torch_dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    manifest = manifest_for_config(config)
    os.makedirs(model_dir, exist_ok=True)
    cfg = dict(config)
    cfg["torch_dtype"] = dtype
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    tensors = ((name, random_tensor(name, spec, seed, device, torch_dtype, std, norm_jitter).cpu())
               for name, spec in manifest.items() if not spec.optional)
    save_file(tensors, os.path.join(model_dir, "model.safetensors"),
              metadata={"format": "pt", "seed": seed})
    return model_dir
