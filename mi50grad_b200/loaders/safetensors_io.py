"""Minimal safetensors reader/writer with no dependency beyond torch/numpy.

The reference parses the format by hand as well (reference:
src/model/weight_loader.py:49-92) and converts BF16 to FP16 on read
(reference: src/model/weight_loader.py:34-46).  Here tensors come back as torch
tensors in their stored dtype unless `bf16_to` asks for a conversion, and the
reader memory-maps the file so a sharded load touches only the bytes it keeps.
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Dict, Iterable, Optional, Tuple

import numpy as np
import torch

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    def __init__(self, path: str, lazy: bool = False):
        """`lazy`: tensors come back as views of the memory-mapped file (copy-on-write private mapping):
        nothing is read until a tensor, or the slice of it that a rank keeps, is actually touched."""
        self.path = str(path)
        self.lazy = lazy
        self.copied_bytes = 0          # bytes materialised by eager reads (stays 0 in lazy mode)
        with open(self.path, "rb") as f:
            (n,) = struct.unpack("<Q", f.read(8))
            self.header = json.loads(f.read(n))
        self.data_offset = 8 + n
        self.metadata = self.header.pop("__metadata__", {})
        self._mm: Optional[mmap.mmap] = None

    def keys(self) -> Iterable[str]:
        return self.header.keys()

    def __contains__(self, key: str) -> bool:
        return key in self.header

    def info(self, key: str) -> Tuple[str, Tuple[int, ...]]:
        e = self.header[key]
        return e["dtype"], tuple(e["shape"])

    def _map(self) -> mmap.mmap:
        if self._mm is None:
            with open(self.path, "rb") as f:
                self._mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_COPY if self.lazy else mmap.ACCESS_READ)
        return self._mm

    def get(self, key: str, bf16_to: Optional[torch.dtype] = None) -> torch.Tensor:
        if key not in self.header:
            raise KeyError(f"Tensor '{key}' not found in {self.path}")
        e = self.header[key]
        if e["dtype"] not in _DTYPES:
            raise ValueError(f"Unsupported dtype: {e['dtype']}")
        dtype, _ = _DTYPES[e["dtype"]]
        start, end = e["data_offsets"]
        if end <= start:
            t = torch.empty(tuple(e["shape"]), dtype=dtype)
        elif self.lazy:
            n = 1
            for d in e["shape"]:
                n *= d
            t = torch.frombuffer(self._map(), dtype=dtype, count=n, offset=self.data_offset + start).reshape(tuple(e["shape"]))
        else:
            buf = self._map()[self.data_offset + start:self.data_offset + end]
            self.copied_bytes += end - start
            t = torch.frombuffer(bytearray(buf), dtype=dtype).reshape(tuple(e["shape"]))
        if dtype == torch.bfloat16 and bf16_to is not None:
            t = t.to(bf16_to)
        return t

    def close(self):
        if self._mm is not None:
            try:
                self._mm.close()
            except BufferError:
                pass                   # lazy tensors still view the mapping: it goes away with the last of them
            self._mm = None


def save_safetensors(path: str, tensors: Dict[str, torch.Tensor],
                     metadata: Optional[Dict[str, str]] = None) -> None:
    header = {}
    if metadata:
        header["__metadata__"] = metadata
    off = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise ValueError(f"Unsupported dtype {t.dtype} for {name}")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


class CheckpointDir:
    """All *.safetensors of a model directory behind one key lookup, using
    model.safetensors.index.json when present (reference:
    src/model/weight_loader.py:264-290)."""

    def __init__(self, model_dir: str, skip_prefixes: Tuple[str, ...] = (), lazy: bool = False):
        self.dir = Path(model_dir)
        self.skip_prefixes = skip_prefixes
        self.lazy = lazy
        self._files: Dict[str, SafetensorsFile] = {}
        self._where: Dict[str, str] = {}
        idx = self.dir / "model.safetensors.index.json"
        if idx.exists():
            self._where.update(json.loads(idx.read_text()).get("weight_map", {}))
        for sf in sorted(self.dir.glob("*.safetensors")):
            f = self._open(sf.name)
            for k in f.keys():
                self._where.setdefault(k, sf.name)

    def _open(self, name: str) -> SafetensorsFile:
        if name not in self._files:
            self._files[name] = SafetensorsFile(self.dir / name, lazy=self.lazy)
        return self._files[name]

    def keys(self):
        return [k for k in self._where if not k.startswith(self.skip_prefixes)] \
            if self.skip_prefixes else list(self._where)

    def __contains__(self, key: str) -> bool:
        return key in self._where

    def get(self, key: str, bf16_to: Optional[torch.dtype] = torch.float16) -> torch.Tensor:
        if key not in self._where:
            raise FileNotFoundError(f"Cannot find tensor: {key}")
        return self._open(self._where[key]).get(key, bf16_to=bf16_to)

    @property
    def copied_bytes(self) -> int:
        return sum(f.copied_bytes for f in self._files.values())

    def shape(self, key: str) -> Tuple[int, ...]:
        return self._open(self._where[key]).info(key)[1]

    def close(self):
        for f in self._files.values():
            f.close()
