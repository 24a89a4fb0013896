"""The description of one step's batch, as the parts and kernels see it.

A step brings, for each of its sequences, a run of new tokens (a whole prompt, or one
token).  The rows of all sequences are packed one after another; only the mixers look
at which sequence and position a row belongs to.  Everything the device needs to know
about the batch lives in ONE int32 buffer that is filled on the host and copied in one
transfer; the fields below are views into it.  A batch can be padded to a fixed number
of rows and sequences (for a captured graph): padding rows carry position -1, which
every kernel that touches the cache skips, and padding changes no result.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..kernels.ops import AttentionBatch


class BatchLayout:
    """Offsets of the fields inside the int32 buffer for given (padded) sizes."""

    def __init__(self, n_tokens: int, n_seqs: int, n_want: int, n_tiles: int, table_widths: Sequence[int],
                 tile_rows: int = 0):
        self.n_tokens, self.n_seqs, self.n_want, self.n_tiles = n_tokens, n_seqs, n_want, n_tiles
        self.tile_rows = tile_rows       # rows of a query tile, as the model's mixers ask for them (0: none)
        self.table_widths = list(table_widths)
        self.fields = {}
        off = 0

        def add(name, n):
            nonlocal off
            self.fields[name] = (off, n)
            off += -(-n // 4) * 4     # keep every field 16-byte aligned

        add("tokens", n_tokens)
        add("token_src", n_tokens)
        add("tok_seq", n_tokens)
        add("tok_pos", n_tokens)
        add("seq_start", n_seqs + 1)
        add("seq_past", n_seqs)
        add("seq_end", n_seqs)
        add("slots", n_seqs)
        add("want_rows", n_want)
        add("tile_seq", n_tiles)
        add("tile_q0", n_tiles)
        for g, w in enumerate(self.table_widths):
            add(f"table{g}", n_seqs * w)
        self.size = max(off, 4)

    def view(self, buf, name):
        off, n = self.fields[name]
        return buf[off:off + n]


@dataclass
class StepBatch:
    layout: BatchLayout
    n_tokens: int                 # rows, padding included
    n_seqs: int                   # sequences, padding included
    real_tokens: int
    real_seqs: int
    n_want: int
    is_decode: bool               # every sequence brings exactly one token
    max_total_len: int            # longest sequence after this step
    tokens: torch.Tensor
    token_src: torch.Tensor       # for tokens taken from an earlier sampling on the device: the row of that result
    tok_seq: torch.Tensor
    tok_pos: torch.Tensor
    seq_start: torch.Tensor
    seq_past: torch.Tensor
    seq_end: torch.Tensor         # past + new: the sequence's length after the step
    slots: torch.Tensor
    want_rows: torch.Tensor
    tile_seq: torch.Tensor
    tile_q0: torch.Tensor
    n_tiles: int
    tables: List[torch.Tensor]    # per kv group: [n_seqs, table_width]
    device: torch.device
    scratch: Dict[str, torch.Tensor] = field(default_factory=dict)   # reusable work buffers, by name
    new_kv: Dict[int, tuple] = field(default_factory=dict)   # run -> (packed rows, key column, value column) of this step
    # run -> the cache write it has put off until the runs that read its keys and values are through (a ring
    # group's rows of earlier steps are still needed by this step's readers); the model calls them
    deferred_writes: Dict[int, object] = field(default_factory=dict)
    cache_owner_of: Dict[int, int] = field(default_factory=dict)     # run -> run whose keys and values it reads
    shared_runs: frozenset = frozenset()                             # runs whose keys and values a later run reads
    status: Optional[torch.Tensor] = None                            # int32 flag kernels set when they give up a wait
    has_past: bool = True                                            # some sequence of the step has earlier positions in the cache

    def attention_batch(self, keys_in_cache: str, window: Optional[int] = None) -> AttentionBatch:
        """keys_in_cache: "past" - new keys are read from the step's packed rows;
        "all" - the step's rows are in the cache already."""
        cached = self.seq_past if keys_in_cache == "past" else self.seq_end
        max_keys = self.max_total_len if window is None else min(self.max_total_len, window)
        return AttentionBatch(self.n_tokens, self.n_seqs, self.tok_seq, self.tok_pos, self.seq_start, self.seq_past,
                              cached, self.tile_seq, self.tile_q0, self.n_tiles, max_keys)

    def scratch_buffer(self, name: str, nbytes: int) -> torch.Tensor:
        """A zero-initialised float32 buffer kept under `name`; its user leaves zero what must start at zero."""
        buf = self.scratch.get(name)
        if buf is None or buf.numel() * 4 < nbytes:
            buf = torch.zeros(-(-nbytes // 4), dtype=torch.float32, device=self.device)
            self.scratch[name] = buf
        return buf


def fill_batch(host: np.ndarray, layout: BatchLayout, *, tokens: Sequence[Sequence[int]], past: Sequence[int],
               slots: Sequence[int], want: Sequence[Sequence[int]], tables: Sequence[np.ndarray],
               token_src: Optional[Sequence[int]] = None):
    """Write the batch description into `host` (int32, layout.size entries).  Returns
    (real_tokens, n_want, n_tiles_used).  token_src: one-token sequences whose token ids are not known
    on the host yet; entry i is the row of an earlier sampling's result that holds sequence i's token."""
    host[:] = 0
    v = lambda name: layout.view(host, name)
    tok, tok_seq, tok_pos = v("tokens"), v("tok_seq"), v("tok_pos")
    tok_pos[:] = -1
    seq_start, seq_past, seq_end, slot_v = v("seq_start"), v("seq_past"), v("seq_end"), v("slots")
    want_rows, tile_seq, tile_q0 = v("want_rows"), v("tile_seq"), v("tile_q0")
    row = 0
    n_want = 0
    n_tiles = 0
    for i, (ids, p) in enumerate(zip(tokens, past)):
        n = len(ids)
        seq_start[i] = row
        tok[row:row + n] = ids
        tok_seq[row:row + n] = i
        tok_pos[row:row + n] = np.arange(p, p + n, dtype=np.int32)
        seq_past[i] = p
        seq_end[i] = p + n
        slot_v[i] = slots[i]
        for w in want[i]:
            if not 0 <= w < n:
                raise ValueError(f"sequence {i}: wanted place {w} is outside its {n} tokens")
            want_rows[n_want] = row + w
            n_want += 1
        if layout.n_tiles and layout.tile_rows:
            for q0 in range(0, n, layout.tile_rows):
                tile_seq[n_tiles] = i
                tile_q0[n_tiles] = q0
                n_tiles += 1
        row += n
    seq_start[len(tokens):] = row      # padding sequences are empty
    if token_src is not None:
        v("token_src")[:len(token_src)] = token_src
    for g, t in enumerate(tables):
        dst = v(f"table{g}").reshape(layout.n_seqs, layout.table_widths[g])
        dst[:t.shape[0]] = t
    return row, n_want, n_tiles


def count_tiles(lengths: Sequence[int], tile_rows: int) -> int:
    """Query tiles of `tile_rows` rows that sequences of these lengths are cut into (a tile never spans two sequences)."""
    return sum(-(-n // tile_rows) for n in lengths) if tile_rows else 0


def batch_from_buffer(dev: torch.Tensor, layout: BatchLayout, *, real_tokens, real_seqs, n_want, n_tiles,
                      is_decode, max_total_len, scratch=None) -> StepBatch:
    v = lambda name: layout.view(dev, name)
    tables = [v(f"table{g}").view(layout.n_seqs, w) for g, w in enumerate(layout.table_widths)]
    return StepBatch(
        layout=layout, n_tokens=layout.n_tokens, n_seqs=layout.n_seqs, real_tokens=real_tokens, real_seqs=real_seqs,
        n_want=n_want, is_decode=is_decode, max_total_len=max_total_len,
        tokens=v("tokens"), token_src=v("token_src"), tok_seq=v("tok_seq"), tok_pos=v("tok_pos"), seq_start=v("seq_start"),
        seq_past=v("seq_past"), seq_end=v("seq_end"), slots=v("slots"), want_rows=v("want_rows")[:n_want],
        tile_seq=v("tile_seq"), tile_q0=v("tile_q0"), n_tiles=n_tiles, tables=tables, device=dev.device,
        scratch=scratch if scratch is not None else {})
