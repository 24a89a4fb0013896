"""Random-weights mode: a model folder from a configuration and a seed.

Writes `config.json` and `model.safetensors` so that every other path of the
library (loader, replay, command line, tests) can use the folder like a real
checkpoint.  The reference can only build unseeded random models in memory
(`rustml/nlp/main/src/core/model.rs:28-71`).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Union

import torch

from ..config.base import architecture_for
from .loader import random_tensor
from .safetensors_io import write_safetensors

_DTYPE_NAMES = {"float32": torch.float32, "bfloat16": torch.bfloat16,
                "fp32": torch.float32, "bf16": torch.bfloat16}


def parse_dtype(name: Union[str, torch.dtype]) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.float32, torch.bfloat16):
            raise ValueError(f"dtype must be float32 or bfloat16, got {name}")
        return name
    try:
        return _DTYPE_NAMES[name]
    except KeyError:
        raise ValueError(f"dtype must be 'float32' or 'bfloat16', got {name!r}") from None


def write_random_model(folder: str, config: Dict[str, Any], seed: int,
                       dtype: Union[str, torch.dtype] = "bfloat16", device="cpu") -> str:
    """Create `folder` with config.json and model.safetensors holding N(0, 0.02) tensors
    (every tensor, norm weights too) in `dtype`, reproducibly from `seed`.  The values depend only
    on (seed, tensor name, element index); `device` only says where they are made (a CUDA device
    makes large models quickly and gives the same file), and `random_model` with the same
    configuration and seed holds the same weights."""
    dtype = parse_dtype(dtype)
    arch = architecture_for(config)
    typed = arch.parse_config(config)
    spec = arch.build_spec(typed)
    os.makedirs(folder, exist_ok=True)
    out = dict(config)
    out.setdefault("architectures", [arch.name])
    out.setdefault("model_type", arch.model_type)
    out["torch_dtype"] = "float32" if dtype is torch.float32 else "bfloat16"
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(out, f, indent=1)
    tensors = {name: random_tensor(t, seed, dtype, device).cpu() for name, t in spec.tensor_specs().items()}
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors,
                      {"format": "pt", "seed": str(seed)})
    return folder
