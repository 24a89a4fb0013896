"""Feed-forward parts.

`GatedMLP`: down(act(gate(x)) * up(x)) (`rustml/nn/main/src/core/feed_forward.rs:151-161`);
sizes and the activation's name are parameters.  gate and up are one product over the
row-concatenated matrices; the activation and the product with `up` run in float32.

Interface of a feed-forward: `forward(x [rows, hidden] normed) -> [rows, hidden]`.  Rows are
independent of each other, so packing and batching never concern it.  Two optional offers, for the split
form of the norms around few-row products (`parts/norm.py`): `takes_deferred_rows` (x may be
`ops.DeferredRows`; it goes into `ops.linear` / `ops.linear_gated` only) and `delivers_branch` (forward takes
`sink` and ends in `ops.linear_branch`).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .registry import BuildContext, register_part
from .spec import PartSpec


class GatedMLP:
    def __init__(self, hidden_size, intermediate_size, activation, w_gate, w_up, w_down):
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"gated_mlp: unknown activation '{activation}', known: {sorted(ops.ACTIVATIONS)}")
        self.hidden_size, self.intermediate_size, self.activation = hidden_size, intermediate_size, activation
        self.w_gate_up = torch.cat([w_gate, w_up], dim=0).contiguous()
        self.w_down = w_down

    takes_deferred_rows = True     # x goes into one product and nowhere else
    delivers_branch = True         # the last product may deliver the result through a stream's sink

    def forward(self, x, sink=None):
        return ops.linear_branch(ops.linear_gated(x, self.w_gate_up, self.activation), self.w_down, sink)


def _build_gated_mlp(spec: PartSpec, ctx: BuildContext) -> GatedMLP:
    p, t = spec.params, spec.tensors
    return GatedMLP(p["hidden_size"], p["intermediate_size"], p["activation"],
                    ctx.tensor(t["gate"]), ctx.tensor(t["up"]), ctx.tensor(t["down"]))


register_part("feed_forward", "gated_mlp", _build_gated_mlp, replace=True)
