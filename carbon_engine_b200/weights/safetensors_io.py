"""A small reader and writer of the safetensors container.

The format is an 8-byte little-endian header length, a JSON header mapping each tensor name to
``dtype``, ``shape`` and ``data_offsets`` (relative to the end of the header), and the raw
little-endian data.  The reference parses the same header by hand (src/weights.rs:389-423) and
finds shards through ``model.safetensors.index.json``'s ``weight_map`` or, failing that, every
``*.safetensors`` file in name order (src/weights.rs:426-452).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One memory-mapped file.  Tensors returned by :meth:`get` alias the mapping."""

    def __init__(self, path: str):
        self.path = path
        self._fh = open(path, "rb")
        size = os.fstat(self._fh.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        (n,) = struct.unpack("<Q", self._fh.read(8))
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: bad header length {n}")
        try:
            header = json.loads(self._fh.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise SafetensorsError(f"{path}: header is not JSON ({exc})") from None
        self._base = 8 + n
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_COPY)
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            dt = _DTYPES.get(meta.get("dtype"))
            if dt is None:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {meta.get('dtype')}")
            shape = tuple(int(s) for s in meta["shape"])
            lo, hi = (int(x) for x in meta["data_offsets"])
            numel = 1
            for s in shape:
                numel *= s
            if hi - lo != numel * torch.empty((), dtype=dt).element_size() or self._base + hi > size:
                raise SafetensorsError(f"{path}: tensor '{name}' has inconsistent offsets")
            self.entries[name] = (dt, shape, lo, hi)

    def names(self) -> List[str]:
        return list(self.entries)

    def get(self, name: str) -> torch.Tensor:
        dt, shape, lo, hi = self.entries[name]
        if hi == lo:
            return torch.empty(shape, dtype=dt)
        flat = torch.frombuffer(self._mm, dtype=dt, count=(hi - lo) // torch.empty((), dtype=dt).element_size(),
                                offset=self._base + lo)
        return flat.view(shape)


def safetensor_files(model_dir: str) -> List[str]:
    """The weight files of a folder, shards first by index then by name (src/weights.rs:426-452)."""
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index, "r", encoding="utf-8") as fh:
            data = json.load(fh)
        wm = data.get("weight_map")
        if not isinstance(wm, dict):
            raise SafetensorsError(f"{index}: weight_map missing")
        return [os.path.join(model_dir, f) for f in sorted(set(wm.values()))]
    files = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors"))
    if not files:
        raise SafetensorsError(f"no .safetensors files found in {model_dir}")
    return [os.path.join(model_dir, f) for f in files]


class TensorDirectory:
    """All tensors of a model folder, by name."""

    def __init__(self, model_dir: str):
        self.files = [SafetensorsFile(p) for p in safetensor_files(model_dir)]
        self._where: Dict[str, SafetensorsFile] = {}
        for f in self.files:
            for n in f.names():
                self._where[n] = f

    def names(self) -> List[str]:
        return list(self._where)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._where[name].entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return self._where[name].entries[name][0]

    def get(self, name: str) -> torch.Tensor:
        return self._where[name].get(name)

    def __contains__(self, name: str) -> bool:
        return name in self._where


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]]) -> None:
    """Write ``(name, tensor)`` pairs; the data of each tensor is aligned to 8 bytes."""
    items = [(n, t.detach().cpu().contiguous()) for n, t in tensors]
    header: Dict[str, Dict] = {}
    offset = 0
    for name, t in items:
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for _, t in items:
            if t.numel():
                fh.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else t.reshape(1).view(torch.uint8).numpy().tobytes())
