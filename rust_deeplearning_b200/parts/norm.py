"""Norms and the residual stream.

`RMSNorm` is y = x / sqrt(mean(x^2) + eps) * (w + offset)
(`rustml/core/main/src/core/tensor/ops.rs:735-743`, offset in
`rustml/nn/main/src/core/rms_norm.rs:43-50`); eps and offset are parameters.

`ResidualStream` keeps the float32 sum of the block outputs.  A block adds a branch
with `add(branch, post_norm)` and asks for `normed(norm)`: when both norms offer
`fused_params()` (scale-only root-mean-square norms: weight, eps, offset), "norm
the branch, add it to the stream, norm the sum for the next part" is ONE kernel
that reads the branch and the stream once.  Any other norm kind (anything with an
`apply`) takes the same route through separate kernels.

Interface of a norm: `apply(x [rows, hidden], out_dtype) -> [rows, hidden]`;
optionally `fused_params() -> ops.NormParams`.
"""
from __future__ import annotations


import torch

from ..kernels import ops
from .registry import BuildContext, register_part
from .spec import PartSpec


class RMSNorm:
    def __init__(self, weight: torch.Tensor, eps: float, offset: float):
        self.weight, self.eps, self.offset = weight, float(eps), float(offset)

    @property
    def params(self) -> ops.NormParams:
        return ops.NormParams(self.weight, self.eps, self.offset)

    def fused_params(self) -> ops.NormParams:
        """A norm of the form x / sqrt(mean(x^2) + eps) * (w + offset) can ride in the fused
        norm-add-norm kernel; any norm part that offers this method with those semantics does."""
        return self.params

    def apply(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        return ops.norm_residual_norm(x, second=self.params, out_dtype=out_dtype)


def _build_rms_norm(spec: PartSpec, ctx: BuildContext) -> RMSNorm:
    p = spec.params
    w = ctx.tensor(spec.tensors["weight"])
    if w.numel() != p["size"]:
        raise ValueError(f"rms_norm: weight of {w.numel()} values for size {p['size']}")
    return RMSNorm(w, p["eps"], p.get("offset", 0.0))


register_part("norm", "rms_norm", _build_rms_norm, replace=True)


def _fusable(norm) -> bool:
    return callable(getattr(norm, "fused_params", None))


class ResidualStream:
    """The running sum x (float32 [rows, hidden]) with at most one branch waiting to be added."""

    def __init__(self, x: torch.Tensor):
        if x.dtype is not torch.float32:
            raise ValueError("the residual stream is float32")
        self.x = x
        self._pending = None     # (branch, post_norm or None)

    def add(self, branch: torch.Tensor, post_norm=None):
        """x <- x + post_norm(branch) (post_norm None: x + branch); done lazily so that the next
        `normed` can fuse it."""
        self._flush()
        self._pending = (branch, post_norm)

    def _flush(self):
        if self._pending is None:
            return
        branch, post = self._pending
        self._pending = None
        if post is None or _fusable(post):
            ops.norm_residual_norm(branch, first=post.fused_params() if post else None, residual=self.x, want_output=False)
        else:
            ops.residual_add_(self.x, post.apply(branch, torch.float32))

    def normed(self, norm, out_dtype: torch.dtype) -> torch.Tensor:
        """norm(x) after any waiting branch has been added."""
        if self._pending is not None and _fusable(norm):
            branch, post = self._pending
            if post is None or _fusable(post):
                self._pending = None
                return ops.norm_residual_norm(branch, first=post.fused_params() if post else None, residual=self.x,
                                              second=norm.fused_params(), out_dtype=out_dtype)
        self._flush()
        return norm.apply(self.x, out_dtype)

    def normed_rows(self, norm, rows: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """norm(x[rows]) for an int32 list of rows."""
        self._flush()
        if _fusable(norm):
            return ops.norm_residual_norm(self.x, second=norm.fused_params(), out_dtype=out_dtype, row_index=rows)
        return norm.apply(ops.convert_rows(self.x, torch.float32, rows), out_dtype)

    def value(self) -> torch.Tensor:
        self._flush()
        return self.x
