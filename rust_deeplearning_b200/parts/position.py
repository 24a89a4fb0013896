"""Position encodings.

`Rotary`: inv_i = theta^(-2i/d), angle = position * inv_i, half-split pairing
(`rustml/nn/main/src/core/rope.rs:93-108, :188-191`).  theta, the head size, how
many of its dimensions rotate and the number of positions are parameters.  The
reference forms theta^(...), the angle and cos/sin in float32; here the angle is
formed in float64 on the host and cos/sin are stored as float32 tables, which
keeps positions in the thousands exact to float32 rounding.

Interface of a position encoding, as an attention mixer uses it:
`rotate(rows, n_heads, n_kv_heads, head_dim, batch)` rotates, in place, the query and
key heads of packed rows [tokens, (n_heads + 2 n_kv_heads) * head_dim] at the rows'
positions.  A part that also offers `tables(device)` and `rotary_dim` lets the
mixer fuse the rotation with the cache write in one kernel.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .registry import BuildContext, register_part
from .spec import PartSpec


class Rotary:
    def __init__(self, theta: float, head_dim: int, rotary_dim: int, max_positions: int, device):
        if rotary_dim % 2 or not 0 < rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim {rotary_dim} must be even and at most head_dim {head_dim}")
        self.theta, self.head_dim, self.rotary_dim, self.max_positions = float(theta), head_dim, rotary_dim, max_positions
        half = rotary_dim // 2
        inv = 1.0 / (torch.tensor(self.theta, dtype=torch.float64) **
                     (2.0 * torch.arange(half, dtype=torch.float64) / rotary_dim))
        ang = torch.arange(max_positions, dtype=torch.float64)[:, None] * inv[None, :]
        self.cos = torch.cos(ang).to(torch.float32).contiguous().to(device)
        self.sin = torch.sin(ang).to(torch.float32).contiguous().to(device)

    def tables(self):
        return self.cos, self.sin

    def rotate(self, rows, n_heads, n_kv_heads, head_dim, batch):
        ops.rope_cache(rows, n_heads, n_kv_heads, head_dim, tok_seq=batch.tok_seq, tok_pos=batch.tok_pos,
                       cos=self.cos, sin=self.sin, rotary_dim=self.rotary_dim)


def _build_rotary(spec: PartSpec, ctx: BuildContext) -> Rotary:
    p = spec.params
    key = ("rotary", p["theta"], p["head_dim"], p["rotary_dim"], p["max_positions"])
    if key not in ctx.shared:     # one table for all layers that share the parameters
        ctx.shared[key] = Rotary(p["theta"], p["head_dim"], p["rotary_dim"], p["max_positions"], ctx.device)
    return ctx.shared[key]


register_part("position", "rotary", _build_rotary, replace=True)
