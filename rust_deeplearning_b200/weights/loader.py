"""Weights by tensor name, checked against the model's description before anything is copied.

The reference looks tensors up one by one and stops at the first missing name
(`rustml/nlp/main/src/core/model.rs:702-707`), skips unmapped tensors with a
warning (`rustml/nlp/main/src/core/weight_map.rs:360-362`) and meets wrong
shapes only later, inside a matrix product.  Here every problem of a file is
found first and reported in one error: missing tensors, unexpected tensors,
wrong shapes and unusable dtypes.
"""
from __future__ import annotations

import fnmatch
import warnings
from typing import Dict, Optional

import torch

from ..parts.spec import ModelSpec, TensorSpec
from . import counter_random
from .safetensors_io import WeightFiles

_FLOAT_FILE_DTYPES = ("F32", "BF16", "F16", "F64")
_INT_FILE_DTYPES = ("I32", "I64")


class WeightError(ValueError):
    """The weight files do not match the model.  Lists every problem found."""

    def __init__(self, where, missing, unexpected, wrong_shape, wrong_dtype):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_dtype = list(wrong_shape), list(wrong_dtype)
        lines = [f"{where}: weights do not match the model"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, want, got in self.wrong_shape:
            lines.append(f"  wrong shape: {name} expected {list(want)}, file has {list(got)}")
        for name, want, got in self.wrong_dtype:
            lines.append(f"  wrong dtype: {name} expected {want}, file has {got}")
        super().__init__("\n".join(lines))


def stored_dtype(spec: TensorSpec, file_dtype: str, compute_dtype: torch.dtype) -> torch.dtype:
    """The dtype a tensor is kept in: matrices in the compute dtype; a small tensor stored in
    32 bits stays 32-bit; integer tables as int32."""
    if spec.kind == "int":
        return torch.int32
    if compute_dtype is torch.float32:
        return torch.float32
    if spec.kind == "vector" and file_dtype in ("F32", "F64"):
        return torch.float32
    return compute_dtype


def check_weights(spec: ModelSpec, files, where: str, strict: bool = True) -> None:
    """Compare the files with the model's description; one WeightError lists everything that is wrong.
    Tensors the model does not read are an error too, unless the architecture declares them
    (`ModelSpec.ignored_tensors`) or `strict` is False, in which case they are listed in a warning
    and skipped, as the reference does (`rustml/nlp/main/src/core/weight_map.rs:360-362`)."""
    wanted = spec.tensor_specs()
    have = set(files.names())
    missing = sorted(n for n in wanted if n not in have)
    unexpected = sorted(n for n in have if n not in wanted
                        and not any(fnmatch.fnmatchcase(n, pat) for pat in spec.ignored_tensors))
    if unexpected and not strict:
        warnings.warn(f"{where}: {len(unexpected)} tensors the model does not read are skipped: " + ", ".join(unexpected))
        unexpected = []
    wrong_shape, wrong_dtype = [], []
    for name, t in wanted.items():
        if name not in have:
            continue
        file_dtype, shape = files.info(name)
        if tuple(shape) != tuple(t.shape):
            wrong_shape.append((name, t.shape, shape))
        allowed = _INT_FILE_DTYPES if t.kind == "int" else _FLOAT_FILE_DTYPES
        if file_dtype not in allowed:
            wrong_dtype.append((name, "/".join(allowed), file_dtype))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(where, missing, unexpected, wrong_shape, wrong_dtype)


def load_weights(spec: ModelSpec, folder: str, compute_dtype: torch.dtype, device, strict: bool = True) -> Dict[str, torch.Tensor]:
    """Every tensor the model names, on `device`, in the dtype it is kept in."""
    files = WeightFiles(folder)
    check_weights(spec, files, folder, strict)
    out = {}
    for name, t in spec.tensor_specs().items():
        file_dtype, _ = files.info(name)
        dtype = stored_dtype(t, file_dtype, compute_dtype)
        out[name] = files.tensor(name).to(device=device, dtype=dtype).contiguous()
    return out


def random_tensor(t: TensorSpec, seed: int, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    """N(0, init_std) values that depend only on (seed, tensor name, element index): the same
    float32 numbers, bit for bit, whether they are made on the host or on a CUDA device
    (`weights/counter_random.py`, `csrc/random_init.cu`), rounded to `dtype` to nearest even.
    The reference's random models are unseeded (`rustml/core/main/src/core/tensor/tensor.rs:217-238`)."""
    if t.kind == "int":
        raise ValueError(f"no random initialisation for integer table '{t.name}'")
    key = counter_random.tensor_key(seed, t.name)
    n = 1
    for d in t.shape:
        n *= int(d)
    if torch.device(device).type == "cuda":
        from ..kernels import ops
        return ops.random_normal(tuple(t.shape), key, t.init_std, dtype, device)
    x = torch.from_numpy(counter_random.normal(n, key, t.init_std)).reshape(tuple(t.shape))
    return x.to(dtype)


def random_weights(spec: ModelSpec, seed: int, compute_dtype: torch.dtype, device,
                   storage_dtype: Optional[torch.dtype] = None) -> Dict[str, torch.Tensor]:
    """Random weights made on `device`, as they would be after writing them in
    `storage_dtype` (default: the compute dtype) and loading them again."""
    storage_dtype = storage_dtype or compute_dtype
    file_dtype = "F32" if storage_dtype is torch.float32 else "BF16"
    out = {}
    for name, t in spec.tensor_specs().items():
        x = random_tensor(t, seed, storage_dtype, device)
        out[name] = x.to(stored_dtype(t, file_dtype, compute_dtype))
    return out
