"""The step function: one batch of sequences, their new tokens, the logits at the wanted places.

The reference's step is `forward_with_cache(input_ids [B, S], cache) -> logits [B, S, V]`
(`rustml/nlp/main/src/api/types.rs:836-837`, `rustml/nlp/main/src/core/model.rs:890-937`):
a rectangle of tokens, one shared past length, logits at every position, and the caller
advances the cache.  Here a step takes sequences of unequal length (whole prompts in one
step, then one token each), runs only the tokens it is given, as one packed batch, on top
of what earlier steps left in the cache, forms logits only where they are wanted, and
advances each sequence's own length.

Single-token steps are replayed from captured CUDA graphs, one per (padded batch size,
context bucket); everything else runs eagerly.  Padding changes no result.
"""
from __future__ import annotations

from typing import Tuple, Dict, List, Optional, Sequence, Union

import numpy as np
import torch

from ..cache.cache import DEFAULT_PAGE_SIZE, Cache
from ..kernels import library, ops
from .batch import BatchLayout, StepBatch, batch_from_buffer, count_tiles, fill_batch


class StepError(ValueError):
    """A step that cannot run: empty sequence, token outside the vocabulary, context too long."""


def _next_pow2(n: int) -> int:
    return 1 << max(0, (n - 1).bit_length())


class _Graph:
    def __init__(self):
        self.graph = None
        self.seen = 0
        self.layout: Optional[BatchLayout] = None
        self.dev: Optional[torch.Tensor] = None
        self.batch: Optional[StepBatch] = None
        self.logits: Optional[torch.Tensor] = None
        self.scratch: Dict[str, torch.Tensor] = {}
        self.kernels = 0          # kernels of the library inside the captured graph


class Engine:
    """A model, its cache and the step function."""

    def __init__(self, model, *, max_tokens: int, max_seqs: Optional[int] = None, max_context: Optional[int] = None,
                 page_size: int = DEFAULT_PAGE_SIZE, use_graphs: bool = True, allocate: bool = True,
                 time_steps: bool = False):
        self.model = model
        self.device = model.device
        max_context = min(max_context or model.max_positions, model.max_positions)
        self.cache = Cache(model.needs(), max_tokens=max_tokens, max_seqs=max_seqs, max_context=max_context,
                           page_size=page_size, dtype=model.dtype, device=model.device, allocate=allocate)
        self.use_graphs = use_graphs and self.device.type == "cuda"
        self._graphs: Dict[tuple, _Graph] = {}
        self._pinned: List[Optional[torch.Tensor]] = [None, None]
        self._pinned_event: List[Optional[torch.cuda.Event]] = [None, None]
        self._flip = 0
        self._scratch: Dict[str, torch.Tensor] = {}
        self.graph_replays = 0
        self.eager_steps = 0
        # time_steps: every step is bracketed by CUDA events on its stream; `step_timings()` reads them
        self.time_steps = time_steps and self.device.type == "cuda"
        self._timed: List[tuple] = []
        # kernels set this word when they give up a bounded wait; pinned host memory, so the host
        # reads it without a device call (after any synchronising read of a step's result)
        self.status = torch.zeros(1, dtype=torch.int32)
        if self.device.type == "cuda":
            self.status = self.status.pin_memory()

    # ---- sequences ----
    def new_sequence(self) -> int:
        return self.cache.alloc_slot()

    def release(self, slot: int):
        self.cache.free_slot(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    def check_status(self):
        """Raise if a kernel of an earlier, completed step reported a fault (call after a synchronising read)."""
        code = int(self.status[0])
        if code:
            self.status[0] = 0
            raise RuntimeError(f"a kernel reported fault {code}: {library.FAULTS.get(code, 'unknown code')}; "
                               f"the results of that step are void")

    # ---- the step ----
    def step(self, slots: Sequence[int], tokens: Optional[Sequence[Sequence[int]]],
             want: Union[str, Sequence[Sequence[int]]] = "last",
             fed: Optional[Tuple[torch.Tensor, Sequence[int]]] = None) -> torch.Tensor:
        """Run `tokens[i]` as the next tokens of sequence `slots[i]`.

        fed (instead of tokens): every sequence brings one token whose id is still on the device:
        (int32 result of an earlier sampling, for each sequence the row of that result).  The host
        need not have read the ids, so this step can be queued while the one before it still runs.

        want: "last", "all", or for each sequence the places among its new tokens whose logits
        are wanted.  Returns float32 logits [wanted places, vocab] on the device, in the order of
        the sequences and of their wanted places.  When it comes from a graph the tensor is
        reused by the next step of the same shape: consume it before stepping again."""
        n = len(slots)
        if fed is not None:
            prev, src = fed
            if tokens is not None or len(src) != n or prev.dtype is not torch.int32 or prev.dim() != 1:
                raise StepError("fed tokens: an int32 vector of sampled ids and one row of it for each sequence, and no host tokens")
            if n and not 0 <= min(src) <= max(src) < prev.numel():
                raise StepError("fed tokens: a row outside the sampled result")
            tokens = [[0]] * n
        if n == 0 or len(tokens) != n:
            raise StepError("a step needs at least one sequence and tokens for each")
        lens = [len(t) for t in tokens]
        if min(lens) < 1:
            raise StepError("a sequence of the step brings no tokens")
        if want == "last":
            want = [[l - 1] for l in lens]
        elif want == "all":
            want = [list(range(l)) for l in lens]
        elif len(want) != n:
            raise StepError("`want` must name places for every sequence")
        for i, (w, l) in enumerate(zip(want, lens)):
            if any(isinstance(x, (bool, float)) or not 0 <= int(x) < l for x in w):
                raise StepError(f"sequence {i}: a wanted place is outside its {l} new tokens (or no whole number)")
        # the ids as arrays, once: checked here, copied into the batch description below (a list of 2,048 ids costs
        # 60-80 us to convert, and the device waits meanwhile)
        tokens = [np.asarray(t).reshape(-1) for t in tokens]
        if any(t.dtype.kind not in "iu" for t in tokens):
            raise StepError("token ids must be whole numbers")
        tokens = [t.astype(np.int64, copy=False) for t in tokens]
        flat = np.concatenate(tokens) if n > 1 else tokens[0]
        if flat.min() < 0 or flat.max() >= self.model.vocab_size:
            raise StepError(f"token id outside the vocabulary of {self.model.vocab_size}")
        past = [self.cache.length(s) for s in slots]
        totals = [p + l for p, l in zip(past, lens)]
        if max(totals) > self.model.max_positions:
            raise StepError(f"a sequence would reach {max(totals)} positions, the model allows {self.model.max_positions}")
        self.cache.reserve(slots, lens)
        if self.time_steps:
            t0 = torch.cuda.Event(enable_timing=True)
            t0.record()
        tables = [g.table_rows(slots) for g in self.cache.kv_groups]
        widths = [g.table_width for g in self.cache.kv_groups]
        is_decode = max(lens) == 1

        if is_decode and self.use_graphs:
            logits = self._graph_step(slots, tokens, past, want, tables, widths, max(totals), fed)
        else:
            n_want = sum(len(w) for w in want)
            tile_rows = self.model.query_tile_rows
            layout = BatchLayout(sum(lens), n, max(n_want, 1), count_tiles(lens, tile_rows), widths, tile_rows)
            host = self._host_buffer(layout.size)
            real_tokens, n_want, n_tiles = fill_batch(host.numpy()[:layout.size], layout, tokens=tokens, past=past,
                                                      slots=slots, want=want, tables=tables,
                                                      token_src=fed[1] if fed is not None else None)
            dev = torch.empty(layout.size, dtype=torch.int32, device=self.device)
            self._upload(dev, host, layout, fed[0] if fed is not None else None, n)
            batch = batch_from_buffer(dev, layout, real_tokens=real_tokens, real_seqs=n, n_want=n_want, n_tiles=n_tiles,
                                      is_decode=is_decode, max_total_len=max(totals), scratch=self._scratch)
            batch.status = self.status
            batch.has_past = max(past) > 0
            logits = self._forward(batch)
            self.eager_steps += 1
        self.cache.advance(slots, lens)
        if self.time_steps:
            t1 = torch.cuda.Event(enable_timing=True)
            t1.record()
            self._timed.append(("decode" if is_decode else "prompt", n, sum(lens), t0, t1))
        return logits

    def step_timings(self) -> List[dict]:
        """Device time of every step since the last call (needs time_steps=True): kind, sequences,
        tokens, milliseconds between CUDA events recorded before and after the step's work."""
        out = []
        for kind, n_seqs, n_tokens, t0, t1 in self._timed:
            t1.synchronize()
            out.append({"kind": kind, "sequences": n_seqs, "tokens": n_tokens, "ms": t0.elapsed_time(t1)})
        self._timed = []
        return out

    # ---- helpers ----
    def _forward(self, batch: StepBatch) -> torch.Tensor:
        """The model on the batch; every kernel it launches reports faults to the engine's status word."""
        with ops.step_status(self.status if self.device.type == "cuda" else None):
            return self.model.forward(batch, self.cache)

    def _host_buffer(self, size: int) -> torch.Tensor:
        self._flip ^= 1
        i = self._flip
        if self._pinned_event[i] is not None:
            self._pinned_event[i].synchronize()     # the earlier copy out of this buffer is done
        buf = self._pinned[i]
        if buf is None or buf.numel() < size:
            buf = torch.empty(max(size, 4096), dtype=torch.int32, pin_memory=self.device.type == "cuda")
            self._pinned[i] = buf
        return buf

    def _upload(self, dev: torch.Tensor, host: torch.Tensor, layout: BatchLayout, sampled: Optional[torch.Tensor] = None, n_fed: int = 0):
        """The batch description goes to the device by a kernel that reads the pinned buffer (a copy engine between
        the kernels of two steps costs several microseconds of hand-over each way); with `sampled`, the first
        n_fed tokens are taken from that device vector on the way: tokens[i] = sampled[token_src[i]]."""
        fed = None
        if sampled is not None:
            fed = (sampled, layout.fields["token_src"][0], layout.fields["tokens"][0], n_fed)
        ops.upload_batch(dev, host, layout.size, fed)
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
            self._pinned_event[self._flip] = ev

    def _graph_step(self, slots, tokens, past, want, tables, widths, max_total, fed=None):
        n = len(slots)
        n_pad = _next_pow2(n)
        len_bucket = min(max(_next_pow2(max_total), 256), self.cache.max_context)
        key = (n_pad, len_bucket)
        g = self._graphs.get(key)
        if g is None:
            g = self._graphs[key] = _Graph()
            g.layout = BatchLayout(n_pad, n_pad, n_pad, 0, widths)
            g.dev = torch.zeros(g.layout.size, dtype=torch.int32, device=self.device)
            g.batch = batch_from_buffer(g.dev, g.layout, real_tokens=n_pad, real_seqs=n_pad, n_want=n_pad, n_tiles=0,
                                        is_decode=True, max_total_len=len_bucket, scratch=g.scratch)
            g.batch.status = self.status
        # logits are formed for every row of the padded batch; the wanted ones are picked afterwards
        all_rows = [[0]] * n
        host = self._host_buffer(g.layout.size)
        fill_batch(host.numpy()[:g.layout.size], g.layout, tokens=tokens, past=past, slots=slots, want=all_rows,
                   tables=tables, token_src=fed[1] if fed is not None else None)
        self._upload(g.dev, host, g.layout, fed[0] if fed is not None else None, n)
        g.seen += 1
        if g.graph is None and g.seen >= 2:
            # the first step of a shape ran eagerly (and warmed the libraries up); capture now
            graph = torch.cuda.CUDAGraph()
            before = library.launch_count
            with torch.cuda.graph(graph):
                g.logits = self._forward(g.batch)
            g.kernels = library.launch_count - before     # captured, not run
            library.launch_count = before
            g.graph = graph
        if g.graph is not None:
            g.graph.replay()
            library.launch_count += g.kernels
            self.graph_replays += 1
            logits = g.logits
        else:
            logits = self._forward(g.batch)
            self.eager_steps += 1
        for i, w in enumerate(want):
            if any(x != 0 for x in w):
                raise StepError(f"sequence {i} brings one token; only place 0 can be wanted")
        picked = [i for i, w in enumerate(want) for _ in w]
        if picked == list(range(len(picked))):
            return logits[:len(picked)]
        return logits[torch.tensor(picked, dtype=torch.long, device=self.device)]
