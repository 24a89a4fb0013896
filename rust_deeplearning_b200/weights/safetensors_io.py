"""Reading and writing safetensors files without any model-side library.

Format (as the reference parses it, `rustml/hub/main/src/core/safetensors.rs:59-121`):
an unsigned 64-bit little-endian header length, a JSON header
`{name: {"dtype", "shape", "data_offsets": [begin, end]}}` with an optional
`__metadata__` entry, then the data; offsets count from the end of the header.
The file is memory-mapped and tensors are handed out as views, so a tensor is
read from disk only when it is copied to the device.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, Iterable, Optional, Tuple

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


# file dtype -> (numpy storage dtype, torch dtype of the view, bytes per element)
_DTYPES = {
    "F32": (np.dtype("<f4"), torch.float32, 4),
    "BF16": (np.dtype("<i2"), torch.bfloat16, 2),
    "F16": (np.dtype("<f2"), torch.float16, 2),
    "F64": (np.dtype("<f8"), torch.float64, 8),
    "I32": (np.dtype("<i4"), torch.int32, 4),
    "I64": (np.dtype("<i8"), torch.int64, 8),
}
_TORCH_TO_FILE = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16",
                  torch.float64: "F64", torch.int32: "I32", torch.int64: "I64"}

_MAX_HEADER = 100 * 1024 * 1024


class SafetensorsFile:
    """One memory-mapped safetensors file."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
        except OSError as e:
            raise SafetensorsError(f"{path}: cannot open ({e.strerror})") from None
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file ({size} bytes)")
        with open(path, "rb") as f:
            (hlen,) = struct.unpack("<Q", f.read(8))
            if hlen > _MAX_HEADER or 8 + hlen > size:
                raise SafetensorsError(f"{path}: header length {hlen} does not fit the file of {size} bytes")
            try:
                header = json.loads(f.read(hlen))
            except (json.JSONDecodeError, UnicodeDecodeError) as e:
                raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", None) or {}
        self.base = 8 + hlen
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        data_size = size - self.base
        spans = []
        for name, info in header.items():
            try:
                dtype, shape, (begin, end) = info["dtype"], tuple(info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed header entry for '{name}'") from None
            whole = lambda v: isinstance(v, int) and not isinstance(v, bool) and v >= 0
            if not (isinstance(info["shape"], list) and all(whole(v) for v in shape) and whole(begin) and whole(end)):
                raise SafetensorsError(f"{path}: malformed header entry for '{name}': sizes and offsets must be whole numbers")
            if not isinstance(dtype, str) or dtype not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {dtype}")
            numel = math.prod(shape)       # Python integers: no overflow
            if not (0 <= begin <= end <= data_size) or end - begin != numel * _DTYPES[dtype][2]:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' ({dtype}{list(shape)}) does not match its data range [{begin}, {end}) "
                    f"in {data_size} bytes of data")
            self.entries[name] = (dtype, shape, begin, end)
            if end > begin:
                spans.append((begin, end, name))
        spans.sort()
        for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
            if b1 < e0:
                raise SafetensorsError(f"{path}: data of '{n0}' and '{n1}' overlap")
        # copy-on-write mapping: the views are writable for torch, the file is never changed
        self._map = np.memmap(path, dtype=np.uint8, mode="c") if size > 0 else None

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def info(self, name: str) -> Tuple[str, Tuple[int, ...]]:
        dtype, shape, _, _ = self.entries[name]
        return dtype, shape

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapped file (no copy)."""
        dtype, shape, begin, end = self.entries[name]
        np_dtype, torch_dtype, _ = _DTYPES[dtype]
        if end == begin:
            return torch.empty(shape, dtype=torch_dtype)
        raw = self._map[self.base + begin:self.base + end]
        if (self.base + begin) % np_dtype.itemsize:
            raw = np.array(raw)  # unaligned data: copy once
        t = torch.from_numpy(raw.view(np_dtype))
        if torch_dtype is torch.bfloat16:
            t = t.view(torch.bfloat16)
        return t.reshape(shape)


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Optional[Dict[str, str]] = None):
    """Write CPU tensors; data is aligned to 8 bytes by padding the header with spaces."""
    header = {}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _TORCH_TO_FILE:
            raise SafetensorsError(f"cannot write tensor '{name}' of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _TORCH_TO_FILE[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-(8 + len(blob)) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.dtype is torch.bfloat16:
                t = t.view(torch.int16)
            f.write(t.numpy().tobytes())
    os.replace(tmp, path)


class WeightFiles:
    """The weight files of a model folder: `model.safetensors`, or the shards that
    `model.safetensors.index.json` names in its `weight_map`."""

    def __init__(self, folder: str):
        self.folder = folder
        single = os.path.join(folder, "model.safetensors")
        index = os.path.join(folder, "model.safetensors.index.json")
        self._files: Dict[str, SafetensorsFile] = {}
        self._where: Dict[str, str] = {}
        if os.path.isfile(single):
            f = SafetensorsFile(single)
            self._files[single] = f
            for n in f.names():
                self._where[n] = single
        elif os.path.isfile(index):
            with open(index) as fh:
                try:
                    weight_map = json.load(fh)["weight_map"]
                except (json.JSONDecodeError, KeyError, TypeError):
                    raise SafetensorsError(f"{index}: no 'weight_map' object") from None
            for shard in sorted(set(weight_map.values())):
                path = os.path.join(folder, shard)
                self._files[path] = SafetensorsFile(path)
            for n, shard in weight_map.items():
                path = os.path.join(folder, shard)
                if n not in self._files[path].entries:
                    raise SafetensorsError(f"{index}: '{n}' is not in shard {shard}")
                self._where[n] = path
        else:
            raise SafetensorsError(f"{folder}: neither model.safetensors nor model.safetensors.index.json")

    def names(self):
        return self._where.keys()

    def info(self, name):
        return self._files[self._where[name]].info(name)

    def tensor(self, name):
        return self._files[self._where[name]].tensor(name)
