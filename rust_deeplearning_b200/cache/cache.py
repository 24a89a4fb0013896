"""The cache: a slot for each sequence, paged keys and values for each layer run, and
per-sequence state of fixed size.

The reference keeps, per layer, K and V of shape [batch, kv_heads, max_seq_len, head_dim]
with ONE length shared by all rows (`rustml/nn/main/src/core/kv_cache.rs:10-17, :97-114`),
so sequences of a batch cannot differ in length and every layer holds the full context.
Here

* a *slot* is one sequence: its length, its pages in every group, its row of state;
* storage is *paged* (pages of `page_size` positions, default 64) and shared by all slots,
  so the cache is sized by the number of tokens that live sequences hold, not by
  slots x longest context;
* layer runs whose mixers declare the same need form a *group* with storage of its own:
  a group that keeps all keys gives a sequence as many pages as its length needs; a group
  with a window of W keys gives it at most ceil((W + 2 * page_size - 2) / page_size) pages,
  used as a ring (position p lives in page-list entry (p / page_size) mod ring);
* state of fixed size lives beside it, [runs in group][slot][*shape], zeroed when a slot
  is handed out.

Freed slots and pages are reused; what a sequence reads is bounded by its length, so stale rows
of an earlier occupant never contribute and nothing is cleared on free.  (Kernels that copy whole
pages may touch such rows, but give them the weight zero; storage starts zero-filled so that
every row they touch holds finite numbers.)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, NamedTuple, Optional, Sequence, Tuple

import numpy as np
import torch


DEFAULT_PAGE_SIZE = 64   # positions a page holds unless an engine is built with another size


class CacheError(RuntimeError):
    """A request the cache cannot serve: no free slot, no free pages, a bad or freed slot."""


@dataclass(frozen=True)
class KVRequirement:
    """Keys and values a mixer keeps per sequence.  window None: all of them.  value_dim: the size of
    a value row where it differs from a key row's (a mixer with compressed or widened values);
    None: the same as head_dim."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    value_dim: Optional[int] = None


@dataclass(frozen=True)
class StateRequirement:
    """State of fixed size a mixer keeps per sequence."""
    shape: Tuple[int, ...]
    dtype: str = "float32"


class RunNeeds(NamedTuple):
    """What one schedule entry needs of the cache."""
    kv: Optional[KVRequirement] = None
    state: Optional[StateRequirement] = None
    reads_cache_of: Optional[int] = None   # schedule entry whose keys and values it reads


class PagePool:
    """Free list of page ids.  Host only."""

    def __init__(self, n_pages: int):
        self.n_pages = n_pages
        self._free = list(range(n_pages - 1, -1, -1))
        self._held = [False] * n_pages

    @property
    def n_free(self):
        return len(self._free)

    def take(self, n: int) -> List[int]:
        if n > len(self._free):
            raise CacheError(f"cache is full: {n} pages needed, {len(self._free)} of {self.n_pages} free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = True
        return out

    def give_back(self, pages: Sequence[int]):
        for p in pages:
            if not (0 <= p < self.n_pages) or not self._held[p]:
                raise CacheError(f"page {p} is given back but not held")
            self._held[p] = False
            self._free.append(p)


def ring_pages_for(window: int, page_size: int) -> int:
    """Entries of a page list a window of `window` keys needs as a ring.  A position may overwrite
    only positions that no later query can see: (ring * page_size) >= window + page_size - 1."""
    return (window + 2 * page_size - 2) // page_size


class KVGroup:
    """Storage of the layer runs that share one KVRequirement."""

    def __init__(self, requirement: KVRequirement, runs: List[int], *, max_tokens: int, max_seqs: int,
                 max_context: int, page_size: int, dtype: torch.dtype, device, allocate: bool = True):
        self.requirement = requirement
        self.runs = list(runs)
        self.page_size = page_size
        context_pages = -(-max_context // page_size)
        if requirement.window is not None and ring_pages_for(requirement.window, page_size) < context_pages:
            self.ring_pages = ring_pages_for(requirement.window, page_size)
            self.is_ring = True
        else:
            self.ring_pages = context_pages
            self.is_ring = False
        self.table_width = self.ring_pages
        total_pages = -(-max_tokens // page_size)
        n_pages = min(total_pages, max_seqs * self.ring_pages)
        self.pool = PagePool(n_pages)
        self.pages: Dict[int, List[int]] = {}          # slot -> page list (ring entries in order of first use)
        k_shape = (len(runs), n_pages, requirement.n_kv_heads, page_size, requirement.head_dim)
        v_shape = k_shape[:-1] + (requirement.value_dim or requirement.head_dim,)
        # zero-filled: kernels that copy whole pages give rows beyond a sequence's length the weight 0,
        # which needs those rows to hold finite numbers (never-written memory may not)
        self.k = torch.zeros(k_shape, dtype=dtype, device=device) if allocate else None
        self.v = torch.zeros(v_shape, dtype=dtype, device=device) if allocate else None

    def pages_needed(self, slot: int, length: int) -> int:
        want = min(-(-length // self.page_size), self.ring_pages)
        return max(0, want - len(self.pages.get(slot, ())))

    def grow(self, slot: int, length: int):
        n = self.pages_needed(slot, length)
        if n:
            self.pages.setdefault(slot, []).extend(self.pool.take(n))

    def release(self, slot: int):
        self.pool.give_back(self.pages.pop(slot, []))

    def table_rows(self, slots: Sequence[int], n_rows: Optional[int] = None) -> np.ndarray:
        out = np.zeros((n_rows or len(slots), self.table_width), dtype=np.int32)
        for i, s in enumerate(slots):
            p = self.pages.get(s, ())
            out[i, :len(p)] = p
        return out

    def nbytes(self):
        return 0 if self.k is None else (self.k.numel() + self.v.numel()) * self.k.element_size()


class StateGroup:
    def __init__(self, requirement: StateRequirement, runs: List[int], max_seqs: int, device, allocate=True):
        self.requirement = requirement
        self.runs = list(runs)
        dtype = getattr(torch, requirement.dtype)
        self.data = torch.zeros((len(runs), max_seqs, *requirement.shape), dtype=dtype, device=device) if allocate else None


class RunCache(NamedTuple):
    """What a mixer gets for one run of its layer in one step."""
    kv_group: Optional[int]         # index into Cache.kv_groups, None if the run keeps no keys
    k: Optional[torch.Tensor]       # [pages, kv_heads, page_size, head_dim]
    v: Optional[torch.Tensor]       # [pages, kv_heads, page_size, value_dim or head_dim]
    page_size: int
    ring_pages: int
    state: Optional[torch.Tensor]   # [max_seqs, *shape], indexed by slot
    owns_kv: bool                   # False: the run reads another run's keys and values
    is_ring: bool = False           # the group keeps a window of keys: a position's row is reused later


class Cache:
    """Slots, pages and state for one model.

    needs: one RunNeeds per schedule entry.  max_tokens: the most tokens live sequences hold at
    any time, each sequence's count rounded up to the page size.  max_seqs: the most sequences
    alive at once (default: max_tokens / page_size).  max_context: the longest sequence."""

    def __init__(self, needs: Sequence[RunNeeds], *, max_tokens: int, max_seqs: Optional[int] = None,
                 max_context: Optional[int] = None, page_size: int = DEFAULT_PAGE_SIZE, dtype: torch.dtype = torch.bfloat16,
                 device="cuda", allocate: bool = True):
        if page_size < 1 or max_tokens < 1:
            raise CacheError("page_size and max_tokens must be positive")
        self.page_size = page_size
        self.max_tokens = -(-max_tokens // page_size) * page_size
        self.max_seqs = max_seqs if max_seqs is not None else max(1, self.max_tokens // page_size)
        self.max_context = min(max_context or self.max_tokens, self.max_tokens)
        self.dtype, self.device = dtype, device
        self.needs = list(needs)

        kv_by_req: Dict[KVRequirement, List[int]] = {}
        state_by_req: Dict[StateRequirement, List[int]] = {}
        for e, n in enumerate(self.needs):
            if n.reads_cache_of is not None:
                src = self.needs[n.reads_cache_of]
                if not (0 <= n.reads_cache_of < e) or src.kv is None or src.reads_cache_of is not None:
                    raise CacheError(f"run {e} reads the cache of run {n.reads_cache_of}, which keeps none of its own")
                if n.kv is not None and (n.kv.n_kv_heads, n.kv.head_dim, n.kv.value_dim or n.kv.head_dim) != \
                        (src.kv.n_kv_heads, src.kv.head_dim, src.kv.value_dim or src.kv.head_dim):
                    raise CacheError(f"run {e} cannot read the cache of run {n.reads_cache_of}: head layout differs")
            elif n.kv is not None:
                kv_by_req.setdefault(n.kv, []).append(e)
            if n.state is not None:
                state_by_req.setdefault(n.state, []).append(e)
        self.kv_groups = [KVGroup(req, runs, max_tokens=self.max_tokens, max_seqs=self.max_seqs,
                                  max_context=self.max_context, page_size=page_size, dtype=dtype, device=device,
                                  allocate=allocate) for req, runs in kv_by_req.items()]
        self.state_groups = [StateGroup(req, runs, self.max_seqs, device, allocate) for req, runs in state_by_req.items()]
        self._kv_of_run = {e: (gi, g.runs.index(e)) for gi, g in enumerate(self.kv_groups) for e in g.runs}
        self._state_of_run = {e: (gi, g.runs.index(e)) for gi, g in enumerate(self.state_groups) for e in g.runs}

        self._free_slots = list(range(self.max_seqs - 1, -1, -1))
        self._live = [False] * self.max_seqs
        self.lengths = [0] * self.max_seqs

    # ---- slots ----
    @property
    def n_free_slots(self):
        return len(self._free_slots)

    def live_slots(self):
        return [s for s, on in enumerate(self._live) if on]

    def alloc_slot(self) -> int:
        if not self._free_slots:
            raise CacheError(f"no free slot: all {self.max_seqs} are in use")
        s = self._free_slots.pop()
        self._live[s] = True
        self.lengths[s] = 0
        for g in self.state_groups:
            if g.data is not None:
                g.data[:, s].zero_()
        return s

    def _check(self, slot: int):
        if not (0 <= slot < self.max_seqs) or not self._live[slot]:
            raise CacheError(f"slot {slot} is not in use")

    def free_slot(self, slot: int):
        self._check(slot)
        for g in self.kv_groups:
            g.release(slot)
        self._live[slot] = False
        self.lengths[slot] = 0
        self._free_slots.append(slot)

    def length(self, slot: int) -> int:
        self._check(slot)
        return self.lengths[slot]

    # ---- growth ----
    def reserve(self, slots: Sequence[int], new_tokens: Sequence[int]):
        """Make room for `new_tokens[i]` more positions of `slots[i]`; all or nothing."""
        if len(set(slots)) != len(slots):
            raise CacheError("a slot is named twice in one step")
        totals = []
        for s, n in zip(slots, new_tokens):
            self._check(s)
            if n < 1:
                raise CacheError(f"slot {s}: a step must bring at least one token")
            total = self.lengths[s] + n
            if total > self.max_context:
                raise CacheError(f"slot {s}: {total} positions exceed the cache's longest context of {self.max_context}")
            totals.append(total)
        for g in self.kv_groups:
            need = sum(g.pages_needed(s, t) for s, t in zip(slots, totals))
            if need > g.pool.n_free:
                raise CacheError(f"cache is full: the step needs {need} more pages of {g.page_size} positions, "
                                 f"{g.pool.n_free} of {g.pool.n_pages} are free (window={g.requirement.window})")
        for g in self.kv_groups:
            for s, t in zip(slots, totals):
                g.grow(s, t)

    def advance(self, slots: Sequence[int], new_tokens: Sequence[int]):
        for s, n in zip(slots, new_tokens):
            self._check(s)
            self.lengths[s] += n

    # ---- views ----
    def run_cache(self, run: int) -> RunCache:
        n = self.needs[run]
        owner = n.reads_cache_of if n.reads_cache_of is not None else run
        kv_group = k = v = None
        page_size, ring, is_ring = self.page_size, 0, False
        if owner in self._kv_of_run:
            kv_group, idx = self._kv_of_run[owner]
            g = self.kv_groups[kv_group]
            k = g.k[idx] if g.k is not None else None
            v = g.v[idx] if g.v is not None else None
            ring, is_ring = g.ring_pages, g.is_ring
        state = None
        if run in self._state_of_run:
            gi, idx = self._state_of_run[run]
            data = self.state_groups[gi].data
            state = data[idx] if data is not None else None
        return RunCache(kv_group, k, v, page_size, ring, state, n.reads_cache_of is None, is_ring)

    def nbytes(self):
        return sum(g.nbytes() for g in self.kv_groups) + sum(
            g.data.numel() * g.data.element_size() for g in self.state_groups if g.data is not None)

    def tokens_held(self) -> int:
        """Tokens held by live sequences, each rounded up to the page size."""
        ps = self.page_size
        return sum(-(-self.lengths[s] // ps) * ps for s in self.live_slots())
