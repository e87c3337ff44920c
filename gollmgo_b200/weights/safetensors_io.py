"""Reader and writer of the safetensors file format.

Format (as the reference reads it, internal/model/weights.go:21-105): eight bytes
of little-endian header length, a JSON object {name: {dtype, shape, data_offsets}}
(the key ``__metadata__`` is skipped), then the raw little-endian tensor data.
A folder is every ``*.safetensors`` file in it, sorted; a name seen twice takes
the later file (internal/model/weights.go:116-163).
"""
from __future__ import annotations

import glob
import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, Tuple

import torch

_DTYPES = {
    "F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
MAX_HEADER = 100 * 1024 * 1024


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int
    end: int


class SafetensorsFile:
    """One file, memory-mapped; ``tensor(name)`` is a view into the mapping."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short for a safetensors file")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > MAX_HEADER or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} is not plausible")
        try:
            header = json.loads(self._f.read(hlen))
        except json.JSONDecodeError as e:
            raise SafetensorsError(f"{path}: header is not JSON: {e}") from None
        self._base = 8 + hlen
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            if info["dtype"] not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name} has unknown dtype {info['dtype']}")
            dt, width = _DTYPES[info["dtype"]]
            shape = tuple(int(s) for s in info["shape"])
            b, e = (int(x) for x in info["data_offsets"])
            n = 1
            for s in shape:
                n *= s
            if e - b != n * width or self._base + e > size:
                raise SafetensorsError(f"{path}: tensor {name} has {e - b} bytes for shape "
                                       f"{list(shape)} of {info['dtype']}")
            self.entries[name] = TensorEntry(name, dt, shape, b, e)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def tensor(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        n = 1
        for s in e.shape:
            n *= s
        if n == 0:
            return torch.empty(e.shape, dtype=e.dtype)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")         # the mapping is read-only; tensors are copied on use
            flat = torch.frombuffer(self._mm, dtype=e.dtype, count=n, offset=self._base + e.begin)
        return flat.view(e.shape)

    def close(self) -> None:
        # tensors handed out keep the mapping alive; dropping our handles is enough
        self._mm = None
        self._f.close()


def open_model_files(model_dir: str) -> Dict[str, Tuple[SafetensorsFile, TensorEntry]]:
    """name -> (file, entry) over every *.safetensors of a folder (or one file)."""
    paths = [model_dir] if os.path.isfile(model_dir) else \
        sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
    if not paths:
        raise SafetensorsError(f"no *.safetensors file in {model_dir}")
    index: Dict[str, Tuple[SafetensorsFile, TensorEntry]] = {}
    for p in paths:
        f = SafetensorsFile(p)
        for name, entry in f.entries.items():
            index[name] = (f, entry)
    return index


def save_file(tensors: Iterable[Tuple[str, torch.Tensor]], path: str, metadata: dict | None = None) -> None:
    """Write tensors (name, tensor) to ``path``; tensors are streamed, not gathered."""
    items = [(n, t.detach().cpu().contiguous()) for n, t in tensors]
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    for name, t in items:
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for _, t in items:
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dtype != torch.bool
                        else t.to(torch.uint8).numpy().tobytes())
