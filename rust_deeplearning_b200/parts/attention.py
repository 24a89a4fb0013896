"""The attention mixer: grouped-query attention over a paged cache.

Per token: q, k, v projections without bias (`rustml/nn/main/src/core/attention.rs:372-374`),
position encoding on q and k (`:394-398`), the new key and value rows go to the cache
(`:401`), scores times `score_scale`, soft-cap, causal and window mask, softmax, P.V
(`:413-446`), output projection (`:448`).  Head counts, head size, score scale, soft-cap,
window and the position encoding are parameters; the mixer does not know the model.

Interface of a mixer:
  needs() -> (KVRequirement | None, StateRequirement | None)  what it keeps per sequence
  forward(x [rows, hidden] normed, batch: StepBatch, cache: RunCache, run: int) -> [rows, hidden]
`cache.owns_kv` False means this run reads the keys and values another run wrote.
Optional offers for the split form of the norms around few-row products (`parts/norm.py`):
`takes_deferred_rows` (x may be `ops.DeferredRows`) and `delivers_branch` (forward takes `sink`).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..cache.cache import KVRequirement, RunCache
from ..kernels import ops
from .registry import BuildContext, build_part, register_part
from .spec import PartSpec


class Attention:
    # the step's batch description lists its prompts cut into tiles of this many query rows (the prefill kernels' tiling)
    query_tile_rows = ops.PREFILL_QUERY_TILE

    def __init__(self, *, hidden_size, n_heads, n_kv_heads, head_dim, score_scale, softcap, window, position,
                 wq, wk, wv, wo):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads cannot share {n_kv_heads} key/value heads")
        if wv.shape[0] != wk.shape[0]:
            raise ValueError("this attention's kernels take key and value rows of one size")
        self.hidden_size, self.n_heads, self.n_kv_heads, self.head_dim = hidden_size, n_heads, n_kv_heads, head_dim
        self.score_scale, self.softcap, self.window = float(score_scale), softcap, window
        self.position = position
        # one product for q, k and v: rows of the three matrices one after another
        self.w_qkv = torch.cat([wq, wk, wv], dim=0).contiguous()
        self.w_q = self.w_qkv[: n_heads * head_dim]       # view, for runs that read another run's cache
        self.w_o = wo
        self.q_width = n_heads * head_dim
        self.kv_width = n_kv_heads * head_dim

    def needs(self):
        return KVRequirement(self.n_kv_heads, self.head_dim, self.window), None

    def _pages(self, batch, cache: RunCache) -> Optional[ops.KVPages]:
        if cache.k is None:
            return None
        return ops.KVPages(cache.k, cache.v, batch.tables[cache.kv_group], cache.page_size, cache.ring_pages)

    def _rotary_tables(self):
        pos = self.position
        if pos is not None and hasattr(pos, "tables") and hasattr(pos, "rotary_dim"):
            return pos.tables(), pos.rotary_dim
        return None, 0

    takes_deferred_rows = True     # x goes into the q/k/v (or q) product and nowhere else
    delivers_branch = True         # the output projection may deliver the result through a stream's sink

    def forward(self, x, batch, cache: RunCache, run: int, sink=None):
        nh, nkv, hd = self.n_heads, self.n_kv_heads, self.head_dim
        pages = self._pages(batch, cache)
        fast = x.dtype is torch.bfloat16 and hd % 16 == 0 and hd <= 256
        fast_decode = fast and nh // nkv <= 8 and cache.page_size % 16 == 0 and cache.page_size <= 64
        common = dict(n_heads=nh, n_kv_heads=nkv, head_dim=hd, score_scale=self.score_scale,
                      softcap=self.softcap, window=self.window)
        tables, rotary_dim = self._rotary_tables()

        if not cache.owns_kv:
            # queries only; keys and values are those of another run of this step
            q = ops.linear(x, self.w_q)
            if self.position is not None:
                if tables is not None:
                    ops.rope_cache(q, nh, 0, hd, tok_seq=batch.tok_seq, tok_pos=batch.tok_pos,
                                   cos=tables[0], sin=tables[1], rotary_dim=rotary_dim)
                else:
                    self.position.rotate(q, nh, 0, hd, batch)
            owner = batch.new_kv.get(cache_owner(batch, run))
            if batch.is_decode or owner is None:
                ab = batch.attention_batch("all", self.window)
                kind = "decode" if (fast_decode and batch.is_decode) else ("prefill" if fast and batch.n_tiles else "plain")
                ctx = ops.attention(q, ab, pages, kind=kind, scratch=lambda n: batch.scratch_buffer("decode", n), status=batch.status, **common)
            else:
                rows, k_col, v_col = owner
                ab = batch.attention_batch("past", self.window)
                ctx = ops.attention(q, ab, pages, new_kv=(rows, k_col, v_col),
                                    kind="prefill" if fast and batch.n_tiles else "plain", **common)
            return ops.linear_branch(ctx, self.w_o, sink)

        qkv = ops.linear(x, self.w_qkv)
        if batch.is_decode and fast_decode and pages is not None and (tables is not None or self.position is None) \
                and rotary_dim % 16 == 0:
            # one kernel rotates, writes the new rows and attends over the cache
            ab = batch.attention_batch("all", self.window)
            ctx = ops.attention(qkv, ab, pages, new_kv=(qkv, self.q_width, self.q_width + self.kv_width), kind="decode",
                                rotate_and_write=(tables[0], tables[1], rotary_dim) if tables is not None else (None, None, 0),
                                scratch=lambda n: batch.scratch_buffer("decode", n), status=batch.status, **common)
        elif batch.is_decode:
            # rotate, write the new row, then read everything from the cache
            if tables is not None or self.position is None:
                ops.rope_cache(qkv, nh, nkv, hd, tok_seq=batch.tok_seq, tok_pos=batch.tok_pos,
                               cos=tables[0] if tables else None, sin=tables[1] if tables else None,
                               rotary_dim=rotary_dim, pages=pages, seq_end=batch.seq_end)
            else:
                self.position.rotate(qkv, nh, nkv, hd, batch)
                ops.rope_cache(qkv, nh, nkv, hd, tok_seq=batch.tok_seq, tok_pos=batch.tok_pos, pages=pages,
                               seq_end=batch.seq_end)
            ab = batch.attention_batch("all", self.window)
            ctx = ops.attention(qkv, ab, pages, kind="decode" if fast_decode else "plain",
                                scratch=lambda n: batch.scratch_buffer("decode", n), status=batch.status, **common)
        else:
            # rotate; attend over the cache (earlier steps) and the packed rows (this step); write.
            # In a ring the write may overwrite rows of earlier steps that this step's early queries still
            # need, so there it comes last; otherwise it rides along with the rotation.
            write_first = pages is not None and (not cache.is_ring or not batch.has_past)
            if tables is not None:
                ops.rope_cache(qkv, nh, nkv, hd, tok_seq=batch.tok_seq, tok_pos=batch.tok_pos,
                               cos=tables[0], sin=tables[1], rotary_dim=rotary_dim,
                               pages=pages if write_first else None, seq_end=batch.seq_end)
            else:
                if self.position is not None:
                    self.position.rotate(qkv, nh, nkv, hd, batch)
                write_first = False
            ab = batch.attention_batch("past", self.window)
            if fast and batch.n_tiles:
                # prompts that start at position 0 read nothing from the cache: the tcgen05 kernel takes them
                kind = "prefill_tc" if (hd % 64 == 0 and not batch.has_past) else "prefill"
            else:
                kind = "plain"
            ctx = ops.attention(qkv, ab, pages, new_kv=(qkv, self.q_width, self.q_width + self.kv_width), kind=kind,
                                status=batch.status, **common)
            if run in batch.shared_runs:
                batch.new_kv[run] = (qkv, self.q_width, self.q_width + self.kv_width)
            if not write_first and pages is not None:
                def write(qkv=qkv, pages=pages):
                    ops.rope_cache(qkv, nh, nkv, hd, tok_seq=batch.tok_seq, tok_pos=batch.tok_pos, pages=pages,
                                   seq_end=batch.seq_end)
                if run in batch.shared_runs and cache.is_ring and batch.has_past:
                    # later runs of this step read this run's rows of earlier steps from the ring: write after them
                    batch.deferred_writes[run] = write
                else:
                    write()
        return ops.linear_branch(ctx, self.w_o, sink)


def cache_owner(batch, run: int) -> int:
    return batch.cache_owner_of[run]


def _build_attention(spec: PartSpec, ctx: BuildContext) -> Attention:
    p, t = spec.params, spec.tensors
    position = build_part("position", p["position"], ctx) if p.get("position") is not None else None
    return Attention(hidden_size=p["hidden_size"], n_heads=p["n_heads"], n_kv_heads=p["n_kv_heads"],
                     head_dim=p["head_dim"], score_scale=p["score_scale"], softcap=p.get("softcap"),
                     window=p.get("window"), position=position,
                     wq=ctx.tensor(t["q"]), wk=ctx.tensor(t["k"]), wv=ctx.tensor(t["v"]), wo=ctx.tensor(t["o"]))


register_part("mixer", "attention", _build_attention, replace=True)
