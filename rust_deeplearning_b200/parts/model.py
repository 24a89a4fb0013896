"""Embedding, output head, the arrangement of a block, and the model that runs a schedule.

Embedding: x[t] = E[id_t] * scale (`rustml/nn/main/src/core/embedding.rs:50-76`,
`rustml/nlp/main/src/core/model.rs:896-900`).  Head: z = n E^T for tied weights
(`model.rs:829-834, :936`) and cap * tanh(z / cap), which the architecture has and the
reference lacks.  Sandwich block: h = x + post(mixer(pre(x))); y = h + post'(ff(pre'(h)))
(`rustml/nn/main/src/core/transformer_block.rs:324-355`); which norms exist is data.

The model runs its schedule: a list of (layer, whose cache it reads).  A layer named
twice runs twice, each run with cache storage of its own.  Logits are formed only at the
rows the step wants (`model.rs:936` forms them at every position).

Interface of a block: `forward(stream: ResidualStream, batch, cache: RunCache, run: int)`;
it adds its branches to the stream.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..cache.cache import RunNeeds
from ..kernels import ops
from .norm import ResidualStream
from .registry import BuildContext, build_part, register_part
from .spec import LayerSpec, ModelSpec


class ScaledEmbedding:
    def __init__(self, table: torch.Tensor, scale: float):
        self.table, self.scale = table, float(scale)
        self.vocab_size, self.hidden_size = table.shape

    def forward(self, tokens: torch.Tensor, status: Optional[torch.Tensor] = None) -> torch.Tensor:
        return ops.embed_rows(self.table, tokens, self.scale, status)


register_part("embedding", "scaled_embedding",
              lambda spec, ctx: ScaledEmbedding(ctx.tensor(spec.tensors["table"]), spec.params.get("scale", 1.0)),
              replace=True)


class LinearHead:
    """float32 logits = soft-cap(n W^T)."""

    def __init__(self, weight: torch.Tensor, softcap: Optional[float]):
        self.weight, self.softcap = weight, softcap

    takes_deferred_rows = True      # n goes into one product and nowhere else

    def forward(self, n) -> torch.Tensor:
        return ops.linear(n, self.weight, out_dtype=torch.float32, softcap=self.softcap)


register_part("head", "linear_head",
              lambda spec, ctx: LinearHead(ctx.tensor(spec.tensors["weight"]), spec.params.get("softcap")),
              replace=True)


class SandwichBlock:
    """pre-norm -> mixer -> optional post-norm -> add; pre-norm -> feed-forward -> optional post-norm -> add."""

    def __init__(self, mixer, feed_forward, norms: Dict[str, object], act_dtype: torch.dtype):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.pre_mixer = norms["pre_mixer"]
        self.post_mixer = norms.get("post_mixer")
        self.pre_ff = norms["pre_feed_forward"]
        self.post_ff = norms.get("post_feed_forward")
        self.act_dtype = act_dtype

    @property
    def first_norm(self):
        """The norm this block asks the stream for first, if its mixer's first product takes the rows in the
        split form (`ops.DeferredRows`); the model tells the block before, so that its last product can prepare them."""
        return self.pre_mixer if getattr(self.mixer, "takes_deferred_rows", False) else None

    def forward(self, stream: ResidualStream, batch, cache, run: int):
        # Parts say what they can do with the split form of the norms (few rows; see ResidualStream):
        # takes_deferred_rows - x goes into ops.linear / ops.linear_gated only; delivers_branch - forward takes
        # `sink` and ends in ops.linear_branch.  Everything else runs through the norm kernels.
        mixer, ff = self.mixer, self.feed_forward
        m_in, m_out = getattr(mixer, "takes_deferred_rows", False), getattr(mixer, "delivers_branch", False)
        f_in, f_out = getattr(ff, "takes_deferred_rows", False), getattr(ff, "delivers_branch", False)
        after, stream.norm_after_block = stream.norm_after_block, None
        x = stream.normed(self.pre_mixer, self.act_dtype, deferred_ok=m_in, upcoming=self.pre_ff if (m_out and f_in) else None)
        sink = stream.branch_sink(self.post_mixer, self.pre_ff) if (m_out and f_in) else None
        a = mixer.forward(x, batch, cache, run, sink=sink) if sink is not None else mixer.forward(x, batch, cache, run)
        stream.add(a, self.post_mixer)
        x = stream.normed(self.pre_ff, self.act_dtype, deferred_ok=f_in, upcoming=after if f_out else None)
        sink = stream.branch_sink(self.post_ff, after) if (f_out and after is not None) else None
        f = ff.forward(x, sink=sink) if sink is not None else ff.forward(x)
        stream.add(f, self.post_ff)


def _build_sandwich(layer: LayerSpec, ctx: BuildContext) -> SandwichBlock:
    mixer = build_part("mixer", layer.mixer, ctx)
    ff = build_part("feed_forward", layer.feed_forward, ctx)
    norms = {role: build_part("norm", s, ctx) for role, s in layer.norms.items()}
    return SandwichBlock(mixer, ff, norms, ctx.dtype)


register_part("block", "sandwich", _build_sandwich, replace=True)


class Model:
    """A model built from a ModelSpec and loaded tensors.  Nothing here names an architecture."""

    def __init__(self, spec: ModelSpec, weights: Dict[str, torch.Tensor], dtype: torch.dtype, device):
        spec.validate()
        self.spec, self.dtype, self.device = spec, dtype, torch.device(device)
        ctx = BuildContext(weights, dtype, self.device)
        self.embedding = build_part("embedding", spec.embedding, ctx)
        keep = {t.name for p in (spec.embedding, spec.final_norm, spec.head) for t in p.tensors.values()}
        self.layers = []
        for layer in spec.layers:
            self.layers.append(build_block(layer, ctx))
            # parts hold what they need (fused copies or the tensors themselves)
            for p in (layer.mixer, layer.feed_forward, *layer.norms.values()):
                for t in p.tensors.values():
                    if t.name not in keep:
                        weights.pop(t.name, None)
        self.final_norm = build_part("norm", spec.final_norm, ctx)
        self.head = build_part("head", spec.head, ctx)
        self.schedule = list(spec.schedule)
        self.cache_owner_of = {e: (s.reads_cache_of if s.reads_cache_of is not None else e)
                               for e, s in enumerate(self.schedule)}
        self.shared_runs = frozenset(s.reads_cache_of for s in self.schedule if s.reads_cache_of is not None)
        # the last run that reads each shared run's keys and values: a cache write that the owner puts off
        # (a ring whose rows this step's readers still need) is done after it
        self.last_reader = {}
        for e, s in enumerate(self.schedule):
            if s.reads_cache_of is not None:
                self.last_reader[s.reads_cache_of] = e
        self.vocab_size, self.hidden_size = spec.vocab_size, spec.hidden_size
        self.max_positions = spec.max_positions
        # Mixers may ask the step for its many-token sequences cut into query tiles of so many rows (a kernel's
        # tiling); the step's batch description then carries the tile lists.  One size per model.
        sizes = {getattr(layer.mixer, "query_tile_rows", 0) or 0 for layer in self.layers if hasattr(layer, "mixer")} - {0}
        if len(sizes) > 1:
            raise ValueError(f"the model's mixers ask for query tiles of different sizes: {sorted(sizes)}")
        self.query_tile_rows = sizes.pop() if sizes else 0

    def needs(self) -> List[RunNeeds]:
        """What each schedule entry needs of the cache."""
        out = []
        for s in self.schedule:
            kv, state = self.layers[s.layer].mixer.needs()
            out.append(RunNeeds(kv, state, s.reads_cache_of))
        return out

    def forward(self, batch, cache) -> torch.Tensor:
        """Runs the batch's tokens through the schedule; float32 logits [wanted rows, vocab]."""
        batch.cache_owner_of, batch.shared_runs = self.cache_owner_of, self.shared_runs
        batch.new_kv.clear()
        stream = ResidualStream(self.embedding.forward(batch.tokens))
        batch.deferred_writes.clear()
        lazy_head = getattr(self.head, "takes_deferred_rows", False)
        for run, entry in enumerate(self.schedule):
            # what the stream will be asked for after this block, where the asker's first product takes the split form
            if run + 1 < len(self.schedule):
                stream.norm_after_block = getattr(self.layers[self.schedule[run + 1].layer], "first_norm", None)
            else:
                stream.norm_after_block = self.final_norm if (lazy_head and batch.n_want) else None
            self.layers[entry.layer].forward(stream, batch, cache.run_cache(run), run)
            stream.norm_after_block = None
            for owner in [o for o in batch.deferred_writes if self.last_reader.get(o, o) <= run]:
                batch.deferred_writes.pop(owner)()
        for write in batch.deferred_writes.values():
            write()
        batch.deferred_writes.clear()
        batch.new_kv.clear()
        if batch.n_want == 0:
            stream.value()
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        n = stream.normed_rows(self.final_norm, batch.want_rows, self.dtype, deferred_ok=lazy_head)
        return self.head.forward(n)


def build_block(layer: LayerSpec, ctx: BuildContext):
    from .registry import _REGISTRY, PartError, registered_parts
    try:
        factory = _REGISTRY["block"][layer.block]
    except KeyError:
        raise PartError(f"no block of kind '{layer.block}'; registered: {registered_parts('block')}") from None
    return factory(layer, ctx)
