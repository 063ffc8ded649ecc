"""Reader and writer for the safetensors container (no third-party package).

Layout (as read by crates/hi-mlx/src/weights.rs:430-440 and
crates/hi-cuda/src/safetensors.rs:181-430): 8-byte little-endian header length,
a JSON header ``{name: {dtype, shape, data_offsets:[begin,end]}, "__metadata__": {...}}``,
then the raw little-endian tensor bytes. Shards are ``*.safetensors`` files sorted by
name; ``model.safetensors.index.json`` (``weight_map``) is honoured when present
(weights.rs:360-420).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "F32": (torch.float32, 4),
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F64": (torch.float64, 8),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class TensorEntry:
    __slots__ = ("name", "dtype_name", "shape", "begin", "end", "shard")

    def __init__(self, name, dtype_name, shape, begin, end, shard):
        self.name, self.dtype_name, self.shape = name, dtype_name, tuple(shape)
        self.begin, self.end, self.shard = begin, end, shard


class Shard:
    """One mmap'd file; tensors are zero-copy views until moved to the device."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short for a safetensors header")
        self._file = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._file.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._file.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})")
        self.data_start = 8 + hlen
        self.metadata = header.pop("__metadata__", {}) or {}
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            try:
                dt, shape, (b, e) = info["dtype"], info["shape"], info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed header entry for tensor '{name}'")
            if dt in _DTYPES:
                n = 1
                for s in shape:
                    n *= int(s)
                if n * _DTYPES[dt][1] != e - b:
                    raise SafetensorsError(
                        f"{path}: tensor '{name}' has shape {shape} ({dt}) but {e - b} bytes")
            if self.data_start + e > size:
                raise SafetensorsError(f"{path}: tensor '{name}' runs past the end of the file")
            self.entries[name] = TensorEntry(name, dt, shape, b, e, self)
        self._mmap = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def tensor(self, entry: TensorEntry) -> torch.Tensor:
        if entry.dtype_name not in _DTYPES:
            raise SafetensorsError(
                f"{self.path}: tensor '{entry.name}' has dtype {entry.dtype_name}; quantized or "
                f"packed weights are not supported")
        dtype, _ = _DTYPES[entry.dtype_name]
        n = entry.end - entry.begin
        if n == 0:
            return torch.empty(entry.shape, dtype=dtype)
        buf = memoryview(self._mmap)[self.data_start + entry.begin: self.data_start + entry.end]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)   # the mapping is read-only and only read
            t = torch.frombuffer(buf, dtype=dtype)
        return t.reshape(entry.shape)


def list_shards(model_dir: str) -> List[str]:
    names = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors"))
    if not names:
        raise SafetensorsError(f"{model_dir}: no .safetensors file")
    return [os.path.join(model_dir, n) for n in names]


class Checkpoint:
    """All tensors of a model folder by name."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        self.shards = [Shard(p) for p in list_shards(model_dir)]
        self.entries: Dict[str, TensorEntry] = {}
        duplicates = []
        index_path = os.path.join(model_dir, "model.safetensors.index.json")
        weight_map = None
        if os.path.isfile(index_path):
            try:
                with open(index_path, "r", encoding="utf-8") as f:
                    weight_map = json.load(f).get("weight_map")
            except json.JSONDecodeError as e:
                raise SafetensorsError(f"{index_path}: not valid JSON ({e})")
            if not isinstance(weight_map, dict):
                raise SafetensorsError(f"{index_path}: no 'weight_map' object")
        by_file = {os.path.basename(s.path): s for s in self.shards}
        if weight_map is not None:
            for name, fname in weight_map.items():
                shard = by_file.get(fname)
                if shard is None or name not in shard.entries:
                    raise SafetensorsError(
                        f"{index_path}: tensor '{name}' is mapped to '{fname}', which does not hold it")
                self.entries[name] = shard.entries[name]
        else:
            for shard in self.shards:
                for name, entry in shard.entries.items():
                    if name in self.entries:
                        duplicates.append(name)
                    self.entries[name] = entry
        if duplicates:
            raise SafetensorsError(
                f"{model_dir}: tensors stored in more than one shard: {sorted(set(duplicates))[:8]}")

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def describe(self, name: str) -> Tuple[str, Tuple[int, ...]]:
        e = self.entries[name]
        return e.dtype_name, e.shape

    def tensor(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        return e.shard.tensor(e)


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] | None = None) -> None:
    """Write one shard. Tensors are stored in name order, 8-byte aligned header."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors.keys())
    blobs = []
    for name in order:
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        if t.dtype == torch.bfloat16:
            raw = t.view(torch.int16).numpy().tobytes()
        elif t.dtype == torch.bool:
            raw = t.to(torch.uint8).numpy().tobytes()
        else:
            raw = t.numpy().tobytes()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hbytes = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hbytes += b" " * ((8 - len(hbytes) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hbytes)))
        f.write(hbytes)
        for raw in blobs:
            f.write(raw)
    os.replace(tmp, path)
