"""Binding of checkpoint tensors to a model, by tensor name.

A model states what it expects as a manifest {name: WeightSpec}.  The loader
checks the whole checkpoint against it first and raises ONE error that lists
every missing tensor, every unexpected tensor and every wrong shape (the
reference finds a missing per-layer tensor only at the first forward pass, and
never checks shapes or dtypes: kernels/gollmgo_model.cu:377-404, 462-473).

Storage rule: floating tensors are kept in bfloat16; a tensor stored in 32-bit
stays 32-bit; integer tables become int32.  In the float32 engine mode every
floating tensor is widened to float32 (exact for bfloat16 and float16).
"""
from __future__ import annotations

import fnmatch
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, Tuple

import torch

from .safetensors_io import open_model_files


class WeightError(ValueError):
    """The checkpoint does not fit the model; the message lists every problem."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_dtype=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = ["checkpoint does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, got, want in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, expected {list(want)}")
        for name, got in self.wrong_dtype:
            lines.append(f"  wrong dtype: {name} is {got}, expected a floating type")
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class WeightSpec:
    shape: Tuple[int, ...]
    kind: str = "float"          # "float" | "int"
    optional: bool = False       # may be absent (e.g. lm_head of a tied model)


# Tensors some exporters add that carry no parameters of the model.
IGNORABLE = ("*.rotary_emb.inv_freq", "*.attn.bias", "*.attn.masked_bias")


def storage_dtype(stored: torch.dtype, kind: str, engine_dtype: torch.dtype) -> torch.dtype:
    if kind == "int":
        return torch.int32
    if engine_dtype == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def check_manifest(manifest: Dict[str, WeightSpec], found: Dict[str, Tuple[Tuple[int, ...], torch.dtype]],
                   ignorable: Iterable[str] = IGNORABLE) -> None:
    missing = [n for n, s in manifest.items() if n not in found and not s.optional]
    unexpected = [n for n in found if n not in manifest
                  and not any(fnmatch.fnmatch(n, pat) for pat in ignorable)]
    wrong_shape, wrong_dtype = [], []
    for n, s in manifest.items():
        if n in found:
            shape, dt = found[n]
            if tuple(shape) != tuple(s.shape):
                wrong_shape.append((n, shape, s.shape))
            if s.kind == "float" and not dt.is_floating_point:
                wrong_dtype.append((n, dt))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(sorted(missing), sorted(unexpected), wrong_shape, wrong_dtype)


def checkpoint_source(model_dir: str, manifest: Dict[str, WeightSpec], engine_dtype: torch.dtype,
                      device) -> Callable[[str], torch.Tensor]:
    """Check the checkpoint in ``model_dir`` against ``manifest``; return ``get(name)``
    that delivers each tensor on ``device`` in its storage dtype (None if optional
    and absent)."""
    index = open_model_files(model_dir)
    check_manifest(manifest, {n: (e.shape, e.dtype) for n, (_, e) in index.items()})

    def get(name: str):
        if name not in index:
            return None
        f, e = index[name]
        spec = manifest[name]
        t = f.tensor(name)
        return t.to(device=device, dtype=storage_dtype(e.dtype, spec.kind, engine_dtype))

    return get
