"""Registries of the parts a model is put together from.

A part is registered under a kind name per role (mixer, feed-forward, norm, position
encoding, block arrangement, embedding, head).  `build_part` looks the kind up and
calls the factory with the part's description and a build context; the factory takes
its tensors from the context by name.  Registering a new kind needs no change to the
library: a test, or a user, can add a mixer of their own and name it in a ModelSpec.
"""
from __future__ import annotations

from typing import Any, Callable, Dict

import torch

from .spec import PartSpec, TensorSpec

ROLES = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head")
_REGISTRY: Dict[str, Dict[str, Callable]] = {r: {} for r in ROLES}


class PartError(ValueError):
    pass


def register_part(role: str, kind: str, factory: Callable, replace: bool = False):
    """factory(spec: PartSpec, ctx: BuildContext) -> the part."""
    if role not in _REGISTRY:
        raise PartError(f"unknown role '{role}', roles are {ROLES}")
    if kind in _REGISTRY[role] and not replace:
        raise PartError(f"{role} '{kind}' is already registered")
    _REGISTRY[role][kind] = factory


def registered_parts(role: str):
    return sorted(_REGISTRY[role])


class BuildContext:
    """What a factory may use: the compute dtype, the device, the loaded tensors by name and a
    place to share derived tables (rotary tables, for one) between parts."""

    def __init__(self, weights: Dict[str, torch.Tensor], dtype: torch.dtype, device):
        self.weights = weights
        self.dtype = dtype
        self.device = device
        self.shared: Dict[Any, Any] = {}

    def tensor(self, t: TensorSpec) -> torch.Tensor:
        try:
            w = self.weights[t.name]
        except KeyError:
            raise PartError(f"tensor '{t.name}' was not loaded") from None
        if tuple(w.shape) != tuple(t.shape):
            raise PartError(f"tensor '{t.name}' has shape {tuple(w.shape)}, expected {tuple(t.shape)}")
        return w


def build_part(role: str, spec: PartSpec, ctx: BuildContext):
    try:
        factory = _REGISTRY[role][spec.kind]
    except KeyError:
        raise PartError(f"no {role} of kind '{spec.kind}'; registered: {registered_parts(role)}") from None
    return factory(spec, ctx)
