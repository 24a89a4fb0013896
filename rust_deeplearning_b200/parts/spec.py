"""The description of a model as data.

An architecture turns its typed configuration into a `ModelSpec`: which mixer,
feed-forward and norms each layer has (with every size and constant as a
parameter), which tensors of the weight file each part reads, and the order in
which layers run.  The parts are built from it through the registries in
`parts.registry`; nothing below this description knows which architecture it
came from.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple


@dataclass(frozen=True)
class TensorSpec:
    """One tensor a part reads from the weight file.

    kind: "matrix"  - kept in the compute dtype (bfloat16 on the fast path, float32 on the 32-bit path)
          "vector"  - small parameter; a tensor stored in 32 bits stays 32-bit, otherwise it follows
                      the compute dtype
          "int"     - integer table, kept as int32
    init_std: standard deviation used by the random-weights mode.
    """
    name: str
    shape: Tuple[int, ...]
    kind: str = "matrix"
    init_std: float = 0.02


@dataclass(frozen=True)
class PartSpec:
    """A part to build: registry key, its sizes and constants, and its tensors by role."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    tensors: Dict[str, TensorSpec] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: the arrangement (`block`) and the parts it arranges."""
    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Dict[str, PartSpec]


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  `layer` indexes `ModelSpec.layers` (a layer may be named twice:
    each run has cache storage of its own).  `reads_cache_of` names an earlier schedule entry
    whose keys and values this run reads instead of writing its own."""
    layer: int
    reads_cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    stop_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    # tensors a checkpoint of this architecture may carry that the model does not read (buffers such as
    # rotary frequencies, a copy of tied weights): names or shell-style patterns; they are skipped silently
    ignored_tensors: Tuple[str, ...] = ()

    def part_specs(self):
        yield self.embedding
        for layer in self.layers:
            yield layer.mixer
            yield layer.feed_forward
            for n in layer.norms.values():
                yield n
        yield self.final_norm
        yield self.head

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        """Every tensor the model reads, by file name.  A name used by two parts (tied
        weights) must be described identically by both."""
        out: Dict[str, TensorSpec] = {}
        for part in self.part_specs():
            for t in part.tensors.values():
                prev = out.get(t.name)
                if prev is not None and (prev.shape != t.shape or prev.kind != t.kind):
                    raise ValueError(f"tensor '{t.name}' is described twice with different shapes or kinds")
                out[t.name] = t
        return out

    def validate(self):
        for e, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"schedule entry {e} names layer {entry.layer}, model has {len(self.layers)}")
            if entry.reads_cache_of is not None and not 0 <= entry.reads_cache_of < e:
                raise ValueError(f"schedule entry {e} reads the cache of entry {entry.reads_cache_of}, "
                                 f"which does not run before it")
