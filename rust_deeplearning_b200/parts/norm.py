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
    """The running sum x (float32 [rows, hidden]) with at most one branch waiting to be added.

    With few rows (decode) the two norms between a branch's last product and the next part's first product
    need no kernel of their own (`ops.DeferredRows`): a part whose last product can deliver its branch in
    the split form asks for `branch_sink(post, then)` and ends in `ops.linear_branch(..., sink)`; a part
    whose first product can take the split form is handed `normed(..., deferred_ok=True)`, which may then
    return `ops.DeferredRows` in place of a tensor.  Both are offers: where one side is missing, where
    the rows are too many or where another norm is asked for than was announced, the stream falls back to
    the kernels of its own, with the same result up to rounding."""

    def __init__(self, x: torch.Tensor):
        if x.dtype is not torch.float32:
            raise ValueError("the residual stream is float32")
        self.x = x
        self._pending = None     # (branch: tensor or ops.Branch, post_norm or None)
        self._operand = None     # (bfloat16 [16, hidden] whose first rows are x times a norm's column factors, that norm)
        self._lent = None        # DeferredRows handed out; x is valid once they have been used
        self.norm_after_block = None     # a hint the model sets: the norm the stream is asked for first after the current block

    # ---- the split form ----
    def _settled(self):
        if self._lent is not None:
            if not self._lent.consumed:
                raise RuntimeError("rows handed out by normed(..., deferred_ok=True) must go into a product (or be "
                                   "materialised) before the stream is used again")
            self._lent = None

    def branch_sink(self, post, then):
        """What `ops.linear_branch` needs to deliver a branch that will be added with `post` and then normed with
        `then`; None where the split form does not apply (the part then returns a plain tensor)."""
        op = self._operand
        if op is None or then is None or op[1] is not then or post is None or not (_fusable(post) and _fusable(then)):
            return None
        return ops.BranchSink(self.x, post.fused_params(), then.fused_params(), op[0])

    def _prepare(self, upcoming, act_dtype):
        """After x has changed: the first half of the operand for `upcoming`, by a kernel of its own."""
        self._operand = None
        if upcoming is not None and _fusable(upcoming) and ops.deferred_ok(self.x.shape[0], self.x.shape[1], act_dtype):
            self._operand = (ops.scaled_rows(self.x, upcoming.fused_params()), upcoming)

    @staticmethod
    def _announced(branch, post, norm) -> bool:
        """Whether a split branch was prepared for exactly these two norms."""
        if post is None or not (_fusable(post) and _fusable(norm)):
            return False
        k = branch.sink
        same = lambda a, b: a.weight is b.weight and a.eps == b.eps and a.offset == b.offset
        return same(k.post, post.fused_params()) and same(k.then, norm.fused_params())

    def _defer(self, branch, upcoming, rows=None):
        out = torch.empty_like(self.x)
        nxt = upcoming if (rows is None and upcoming is not None and _fusable(upcoming)) else None
        operand = torch.empty_like(branch.sink.operand) if nxt is not None else None
        d = ops.DeferredRows(branch, out, nxt.fused_params() if nxt is not None else None, operand, rows)
        self.x = out
        self._operand = (operand, nxt) if nxt is not None else None
        self._lent = d
        return d

    # ---- the stream ----
    def add(self, branch, post_norm=None):
        """x <- x + post_norm(branch) (post_norm None: x + branch); done lazily so that the next
        `normed` can fuse it.  branch: a tensor, or the `ops.Branch` a sink produced."""
        self._settled()
        self._flush()
        self._pending = (branch, post_norm)

    def _flush(self):
        if self._pending is None:
            return
        branch, post = self._pending
        self._pending = None
        self._operand = None
        if isinstance(branch, ops.Branch):
            ops.add_branch_(branch)
        elif post is None or _fusable(post):
            ops.norm_residual_norm(branch, first=post.fused_params() if post else None, residual=self.x, want_output=False)
        else:
            ops.residual_add_(self.x, post.apply(branch, torch.float32))

    def normed(self, norm, out_dtype: torch.dtype, deferred_ok: bool = False, upcoming=None):
        """norm(x) after any waiting branch has been added.  deferred_ok: the caller's first product takes
        `ops.DeferredRows`.  upcoming: the norm the stream will be asked for after the next branch, if the
        caller knows it and both sides of that branch can use the split form."""
        self._settled()
        if self._pending is not None and isinstance(self._pending[0], ops.Branch):
            branch, post = self._pending
            if deferred_ok and out_dtype is branch.dtype and self._announced(branch, post, norm):
                self._pending = None
                return self._defer(branch, upcoming)
        elif self._pending is not None and _fusable(norm):
            branch, post = self._pending
            if post is None or _fusable(post):
                self._pending = None
                y = ops.norm_residual_norm(branch, first=post.fused_params() if post else None, residual=self.x,
                                           second=norm.fused_params(), out_dtype=out_dtype)
                self._prepare(upcoming, out_dtype)
                return y
        self._flush()
        self._prepare(upcoming, out_dtype)
        return norm.apply(self.x, out_dtype)

    def normed_rows(self, norm, rows: torch.Tensor, out_dtype: torch.dtype, deferred_ok: bool = False):
        """norm(x[rows]) for an int32 list of rows."""
        self._settled()
        if self._pending is not None and isinstance(self._pending[0], ops.Branch):
            branch, post = self._pending
            if deferred_ok and out_dtype is branch.dtype and rows.numel() <= ops.DEFERRED_MAX_ROWS and self._announced(branch, post, norm):
                self._pending = None
                return self._defer(branch, None, rows)
        self._flush()
        if _fusable(norm):
            return ops.norm_residual_norm(self.x, second=norm.fused_params(), out_dtype=out_dtype, row_index=rows)
        return norm.apply(ops.convert_rows(self.x, torch.float32, rows), out_dtype)

    def value(self) -> torch.Tensor:
        self._settled()
        self._flush()
        return self.x
