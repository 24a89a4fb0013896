"""Typed entry points of the CUDA kernels, over torch tensors.

Each function checks devices, dtypes, shapes and contiguity, launches on torch's
current stream and returns torch tensors.  There is no other implementation
behind these names: on a machine without the library or without a GPU they
raise.  Parts call them as `ops.<name>` (attribute lookup at call time).
"""
from __future__ import annotations

import ctypes
import functools
import os
from typing import NamedTuple, Optional, Tuple

import torch

from . import library
from .library import AttentionArgs, KernelError, SamplingArgs

# Names of gated activations -> the codes of `csrc/api.h` (RDL_ACT_*).  The functions themselves are in
# `csrc/activations.cuh`, the one place every kernel with a gated epilogue takes them from.
ACTIVATIONS = {"gelu_pytorch_tanh": 0, "gelu_tanh": 0, "silu": 1}

# The status word of the step that is running: every kernel that can report a fault (a token id
# outside the table, a bounded wait that ran out) gets it unless the caller passes one of its own.
# The engine sets it around a step; parts need not know about it.
_step_status: Optional[torch.Tensor] = None


class step_status:
    """`with ops.step_status(word): ...` - kernels launched inside report their faults to `word` (int32[1])."""

    def __init__(self, word: Optional[torch.Tensor]):
        self.word = word

    def __enter__(self):
        global _step_status
        self.before, _step_status = _step_status, self.word
        return self.word

    def __exit__(self, *exc):
        global _step_status
        _step_status = self.before
        return False


def _status(status: Optional[torch.Tensor]):
    status = status if status is not None else _step_status
    return ctypes.c_void_p(status.data_ptr()) if status is not None else None


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype is torch.float32:
        return 0
    if t.dtype is torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _stream(t: torch.Tensor):
    if not t.is_cuda:
        raise KernelError("kernels run on CUDA tensors only; there is no CPU path")
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _need(cond, msg):
    if not cond:
        raise KernelError(msg)


def _dense(t, name):
    _need(t.is_contiguous(), f"{name} must be contiguous")
    return t


def _int32(t, name, n=None):
    _need(t.dtype is torch.int32 and t.is_contiguous(), f"{name} must be a contiguous int32 tensor")
    if n is not None:
        _need(t.numel() >= n, f"{name} holds {t.numel()} entries, {n} are needed")
    return t


# ------------------------------------------------------------------------------------------
# row-wise kernels
# ------------------------------------------------------------------------------------------

def embed_rows(table: torch.Tensor, ids: torch.Tensor, scale: float, status: Optional[torch.Tensor] = None):
    """float32 rows `table[ids] * scale`.  An id outside the table poisons its row with NaN and
    sets `status[0]` (int32) if given."""
    _dense(table, "embedding table")
    _int32(ids, "ids")
    V, H = table.shape
    T = ids.numel()
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    library.check(library.load().rdl_embed_rows(_ptr(out), _ptr(table), _dtype_code(table), _ptr(ids), float(scale),
                                                T, H, V, _status(status), _stream(table)))
    return out


class NormParams(NamedTuple):
    weight: torch.Tensor
    eps: float
    offset: float


def norm_residual_norm(x: torch.Tensor, *, first: Optional[NormParams] = None, residual: Optional[torch.Tensor] = None,
                       second: Optional[NormParams] = None, out_dtype: Optional[torch.dtype] = None,
                       row_index: Optional[torch.Tensor] = None, want_output: bool = True):
    """t = first ? rms_norm(x; first) : x;  h = residual + t (written back to `residual`, float32)
    or t;  returns second ? rms_norm(h; second) : h in `out_dtype`, or None if not wanted.
    rms_norm(v; w, eps, off) = v / sqrt(mean(v^2) + eps) * (w + off), statistics in float32."""
    _dense(x, "x")
    _need(x.dim() == 2, "x must be [rows, hidden]")
    H = x.shape[1]
    rows = row_index.numel() if row_index is not None else x.shape[0]
    if row_index is not None:
        _int32(row_index, "row_index")
    for p, name in ((first, "first"), (second, "second")):
        if p is not None:
            _need(p.weight.is_contiguous() and p.weight.numel() == H, f"{name} norm weight must hold {H} values")
    if residual is not None:
        _need(residual.dtype is torch.float32 and residual.is_contiguous() and tuple(residual.shape) == (rows, H),
              "residual must be a contiguous float32 [rows, hidden] tensor")
    y = torch.empty((rows, H), dtype=out_dtype or x.dtype, device=x.device) if want_output else None
    _need(y is not None or residual is not None, "norm_residual_norm: nothing to write")
    library.check(library.load().rdl_norm_residual_norm(
        _ptr(x), _dtype_code(x), _ptr(row_index),
        _ptr(first.weight) if first else None, _dtype_code(first.weight) if first else 0,
        float(first.eps) if first else 0.0, float(first.offset) if first else 0.0,
        _ptr(residual),
        _ptr(second.weight) if second else None, _dtype_code(second.weight) if second else 0,
        float(second.eps) if second else 0.0, float(second.offset) if second else 0.0,
        _ptr(y), _dtype_code(y) if y is not None else 0, rows, H, _stream(x)))
    return y


def gated_activation(gate_up: torch.Tensor, activation: str):
    """[rows, 2I] -> [rows, I]: act(gate_up[:, :I]) * gate_up[:, I:], computed in float32."""
    _dense(gate_up, "gate_up")
    _need(activation in ACTIVATIONS, f"unknown activation '{activation}', known: {sorted(ACTIVATIONS)}")
    rows, two_i = gate_up.shape
    _need(two_i % 2 == 0, "gate_up must have an even width")
    out = torch.empty((rows, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    library.check(library.load().rdl_gated_activation(_ptr(out), _ptr(gate_up), _dtype_code(gate_up),
                                                      ACTIVATIONS[activation], rows, two_i // 2, _stream(gate_up)))
    return out


def softcap_(z: torch.Tensor, cap: float):
    """In place on float32: cap * tanh(z / cap)."""
    _need(z.dtype is torch.float32 and z.is_contiguous(), "softcap_ takes a contiguous float32 tensor")
    library.check(library.load().rdl_softcap_inplace(_ptr(z), z.numel(), float(cap), _stream(z)))
    return z


def residual_add_(residual: torch.Tensor, x: torch.Tensor):
    _need(residual.dtype is torch.float32 and residual.is_contiguous() and x.is_contiguous()
          and residual.shape == x.shape, "residual_add_ takes a float32 residual and an addend of the same shape")
    library.check(library.load().rdl_residual_add(_ptr(residual), _ptr(x), _dtype_code(x), residual.numel(), _stream(x)))
    return residual


def convert_rows(x: torch.Tensor, out_dtype: torch.dtype, row_index: Optional[torch.Tensor] = None):
    """Rows of x (all, or those `row_index` names) converted to `out_dtype`."""
    _dense(x, "x")
    rows = row_index.numel() if row_index is not None else x.shape[0]
    if row_index is not None:
        _int32(row_index, "row_index")
    out = torch.empty((rows, x.shape[1]), dtype=out_dtype, device=x.device)
    library.check(library.load().rdl_convert_rows(_ptr(out), _dtype_code(out), _ptr(x), _dtype_code(x), _ptr(row_index),
                                                  rows, x.shape[1], _stream(x)))
    return out


# ------------------------------------------------------------------------------------------
# matrix products
# ------------------------------------------------------------------------------------------

SKINNY_MAX_ROWS = 16     # up to this many rows the weight-streaming kernel runs; above, the tcgen05 kernel
# "tcgen05": the library's own TMA + tcgen05 kernel for products with many rows; "cublas": the library
# product through torch (kept for comparison; set RDL_PREFILL_GEMM=cublas)
PREFILL_GEMM = os.environ.get("RDL_PREFILL_GEMM", "tcgen05")


def _bf16_ok(x, weight):
    return (x.dtype is torch.bfloat16 and weight.dtype is torch.bfloat16 and x.shape[1] % 8 == 0
            and x.is_contiguous() and weight.is_contiguous() and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def _skinny_ok(x, weight):
    return _bf16_ok(x, weight) and x.shape[0] <= SKINNY_MAX_ROWS


TC_MIN_ROWS = 128        # a tcgen05 tile holds 128 rows; between 17 and 127 rows a library product stands


def _own_bf16_kernel(x, weight):
    """Few rows: the weight-streaming kernel.  A tile's worth of rows or more: the tcgen05 kernel.
    In between a 128-row tile would be mostly empty and too few blocks would stream the weights,
    so the library product (cuBLAS through torch) takes those."""
    if not _bf16_ok(x, weight):
        return False
    rows = x.shape[0]
    return rows <= SKINNY_MAX_ROWS or (rows >= TC_MIN_ROWS and PREFILL_GEMM == "tcgen05")


def _gemm_bf16(x, weight, n_out, out_dtype, gated, activation, softcap, status):
    """The library's own bfloat16 products: weight streaming for few rows, tcgen05 for many."""
    out = torch.empty((x.shape[0], n_out), dtype=out_dtype, device=x.device)
    lib = library.load()
    if x.shape[0] <= SKINNY_MAX_ROWS:
        library.check(lib.rdl_gemm_skinny(_ptr(out), _dtype_code(out), _ptr(x), _ptr(weight), x.shape[0], n_out, x.shape[1],
                                          int(gated), activation, float(softcap or 0.0), _status(status), _stream(x)))
    else:
        library.check(lib.rdl_gemm_tc(_ptr(out), _dtype_code(out), _ptr(x), _ptr(weight), x.shape[0], n_out, x.shape[1],
                                      int(gated), activation, float(softcap or 0.0), _status(status), _stream(x)))
    return out


# ------------------------------------------------------------------------------------------
# deferred norms: "norm the branch, add it to the stream, norm the sum" without a kernel of its own
# ------------------------------------------------------------------------------------------
# With up to DEFERRED_MAX_ROWS rows (decode) the two norms between the last product of a branch (P) and the
# first product after them (C) cost more than the products: a kernel that waits for whole rows twice.  The
# norms are scalings by one number a row and one number a column, so they can be split (the algebra stands in
# csrc/api.h at DeferredNormArgs): P's epilogue applies the column factors and writes partial sums of squares,
# C multiplies an operand of 2 x 8 rows (the stream's rows and the branch's rows, both with the second norm's
# column factors) and applies the row factors in its epilogue.  Three small types carry this through the parts.

DEFERRED_MAX_ROWS = 8
# A very wide product (the output head) runs for most of its time in its steady state, where multiplying 16 rows
# instead of 8 costs more than the two small kernels it saves (256,000 outputs: 230 against 165 us): its rows are
# made into a tensor first.
DEFERRED_MAX_OUTPUTS = 65536
DEFERRED_NORMS = os.environ.get("RDL_DEFERRED_NORMS", "1") != "0"     # 0: the norm kernels everywhere, for comparison


class BranchSink(NamedTuple):
    """What the last product of a branch is given so that it can deliver its result in the split form."""
    residual: torch.Tensor     # float32 [rows, width]: the stream the branch will be added to
    post: NormParams           # the norm of the branch before the sum
    then: NormParams           # the norm the sum is asked for next
    operand: torch.Tensor      # bfloat16 [16, width]: its first rows are (by the time the product runs) residual * (then.weight + then.offset)


class Branch:
    """A branch delivered through a BranchSink: a' = y (post.weight + post.offset) [rows, width] in bfloat16,
    the partial sums [units, 8, 4] and, in the operand's second half (`second_half_row`), a' (then.weight + then.offset)."""

    def __init__(self, sink: BranchSink, values: torch.Tensor, sums: torch.Tensor):
        self.sink, self.values, self.sums = sink, values, sums
        self.shape, self.dtype, self.device = values.shape, values.dtype, values.device


class DeferredRows:
    """Stands for then(residual + post(branch)) [rows, width], or for `row_index`'s rows of it, in the act dtype.
    `linear` and `linear_gated` take it in place of a tensor; `materialise()` gives the tensor.  Its first
    use also writes the updated stream to `residual_out` and, if `next_norm` is given, the first half of
    `next_operand` (the rows of the updated stream times that norm's column factors)."""

    def __init__(self, branch: Branch, residual_out: torch.Tensor, next_norm: Optional[NormParams] = None,
                 next_operand: Optional[torch.Tensor] = None, row_index: Optional[torch.Tensor] = None):
        self.branch, self.residual_out = branch, residual_out
        self.next_norm, self.next_operand, self.row_index = next_norm, next_operand, row_index
        rows = row_index.numel() if row_index is not None else branch.shape[0]
        self.shape, self.dtype, self.device = (rows, branch.shape[1]), branch.dtype, branch.device
        self.consumed = False

    def _args(self) -> "library.DeferredNormArgs":
        b, k = self.branch, self.branch.sink
        d = library.DeferredNormArgs()
        d.mode = library.NORM_DEFERRED
        d.sums, d.n_sums = b.sums.data_ptr(), b.sums.shape[0]
        d.eps1, d.eps2 = float(k.post.eps), float(k.then.eps)
        d.n_out = self.shape[0]
        if self.row_index is not None:
            d.row_index = self.row_index.data_ptr()
        if not self.consumed:
            d.branch_in, d.residual_in, d.residual_out = b.values.data_ptr(), k.residual.data_ptr(), self.residual_out.data_ptr()
            if self.next_norm is not None:
                w = self.next_norm.weight
                d.w_next, d.w_next_dtype, d.off_next = w.data_ptr(), _dtype_code(w), float(self.next_norm.offset)
                d.scaled_next = self.next_operand.data_ptr()
        return d

    def materialise(self) -> torch.Tensor:
        b, k = self.branch, self.branch.sink
        rows, width = b.shape
        if not self.consumed:
            n = self.next_norm
            library.check(library.load().rdl_stream_rows(
                _ptr(b.sums), b.sums.shape[0], float(k.post.eps), _ptr(b.values), _ptr(k.residual), _ptr(self.residual_out),
                _ptr(n.weight) if n else None, _dtype_code(n.weight) if n else 0, float(n.offset) if n else 0.0,
                _ptr(self.next_operand) if n else None, rows, width, _stream(b.values)))
            self.consumed = True
        return norm_residual_norm(self.residual_out, second=k.then, out_dtype=self.dtype, row_index=self.row_index)


def add_branch_(branch: Branch) -> torch.Tensor:
    """residual += s1 * a' in place: a split branch that no product takes further."""
    k = branch.sink
    rows, width = branch.shape
    library.check(library.load().rdl_stream_rows(_ptr(branch.sums), branch.sums.shape[0], float(k.post.eps), _ptr(branch.values),
                                                 _ptr(k.residual), _ptr(k.residual), None, 0, 0.0, None, rows, width,
                                                 _stream(branch.values)))
    return k.residual


def scaled_rows(residual: torch.Tensor, norm: NormParams, operand: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The first half of a deferred product's operand, made by a kernel of its own (the first link of a chain):
    rows 0.. of a bfloat16 [16, width] buffer = residual * (norm.weight + norm.offset)."""
    rows, width = residual.shape
    _need(residual.dtype is torch.float32 and residual.is_contiguous() and rows <= DEFERRED_MAX_ROWS, "scaled_rows: up to 8 contiguous float32 rows")
    if operand is None:
        operand = torch.empty((2 * DEFERRED_MAX_ROWS, width), dtype=torch.bfloat16, device=residual.device)
    library.check(library.load().rdl_stream_rows(None, 0, 0.0, None, _ptr(residual), None, _ptr(norm.weight), _dtype_code(norm.weight),
                                                 float(norm.offset), _ptr(operand), rows, width, _stream(residual)))
    return operand


def second_half_row(rows: int) -> int:
    """The operand's row at which the branch's half starts: 8, or 4 with up to 4 rows (the two halves then share one
    8-row fragment of the tensor-core product and cost what 8 plain rows cost)."""
    return 4 if rows <= 4 else DEFERRED_MAX_ROWS


def deferred_ok(rows: int, width: int, dtype: torch.dtype) -> bool:
    """Whether rows of this many and this width can take the split form at all."""
    return DEFERRED_NORMS and dtype is torch.bfloat16 and 0 < rows <= DEFERRED_MAX_ROWS and width % 8 == 0


def linear_branch(x: torch.Tensor, weight: torch.Tensor, sink: Optional[BranchSink], status: Optional[torch.Tensor] = None):
    """x W^T as a branch of a residual stream: a `Branch` where the split form applies, else the plain result."""
    if sink is None or not (_skinny_ok(x, weight) and deferred_ok(x.shape[0], weight.shape[0], x.dtype)
                            and tuple(sink.residual.shape) == (x.shape[0], weight.shape[0])):
        return linear(x, weight, status=status)
    rows, width = x.shape[0], weight.shape[0]
    for p in (sink.post, sink.then):
        _need(p.weight.is_contiguous() and p.weight.numel() == width, f"a norm's weight must hold {width} values")
    _need(sink.operand.dtype is torch.bfloat16 and tuple(sink.operand.shape) == (2 * DEFERRED_MAX_ROWS, width)
          and sink.operand.is_contiguous(), "the sink's operand must be bfloat16 [16, width]")
    values = torch.empty((rows, width), dtype=torch.bfloat16, device=x.device)
    sums = torch.empty(((width + 15) // 16, 8, 4), dtype=torch.float32, device=x.device)
    d = library.DeferredNormArgs()
    d.mode = library.NORM_BRANCH
    d.sums = sums.data_ptr()
    d.residual = sink.residual.data_ptr()
    d.w1, d.w1_dtype, d.off1 = sink.post.weight.data_ptr(), _dtype_code(sink.post.weight), float(sink.post.offset)
    d.w2, d.w2_dtype, d.off2 = sink.then.weight.data_ptr(), _dtype_code(sink.then.weight), float(sink.then.offset)
    d.branch, d.scaled = values.data_ptr(), sink.operand.data_ptr() + second_half_row(rows) * width * 2
    library.check(library.load().rdl_gemm_skinny_norm(None, 0, _ptr(x), _ptr(weight), rows, width, x.shape[1], 0, 0, 0.0,
                                                      ctypes.byref(d), _status(status), _stream(x)))
    return Branch(sink, values, sums)


def _linear_deferred(x: DeferredRows, weight: torch.Tensor, n_out: int, out_dtype, gated: bool, activation: int, softcap, status):
    """The product after a deferred norm, or None if this weight cannot take it."""
    width = x.branch.shape[1]
    if not (weight.dtype is torch.bfloat16 and weight.is_contiguous() and weight.data_ptr() % 16 == 0 and weight.shape[1] == width):
        return None
    if n_out > DEFERRED_MAX_OUTPUTS:
        return None
    out = torch.empty((x.shape[0], n_out), dtype=out_dtype, device=weight.device)
    d = x._args()
    library.check(library.load().rdl_gemm_skinny_norm(_ptr(out), _dtype_code(out), _ptr(x.branch.sink.operand), _ptr(weight),
                                                      x.branch.shape[0], n_out, width, int(gated), activation, float(softcap or 0.0),
                                                      ctypes.byref(d), _status(status), _stream(out)))
    x.consumed = True
    return out


def linear(x, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           softcap: Optional[float] = None, status: Optional[torch.Tensor] = None):
    """x [rows, in] times weight [out, in] transposed; optionally cap * tanh(. / cap) on the result.
    x may be `DeferredRows` (the rows after a deferred norm).

    float32: the library's own FMA kernel (no tensor cores, no reduced-precision mode).
    bfloat16: up to 16 rows (decode) the weight-streaming tensor-core kernels, from 128 rows the TMA +
    tcgen05 kernels, all with float accumulation and the soft-cap in their epilogue.  17 to 127 rows, and
    operands that do not meet the alignment rules, go to a library product (cuBLAS through torch), which
    is what the reference's engine uses for all its products."""
    if isinstance(x, DeferredRows):
        _need(softcap is None or out_dtype is torch.float32, "linear: the soft-cap is applied to float32 results")
        out = _linear_deferred(x, weight, weight.shape[0], out_dtype or x.dtype, False, 0, softcap, status)
        if out is not None:
            return out
        x = x.materialise()
    _need(x.dim() == 2 and weight.dim() == 2 and x.shape[1] == weight.shape[1],
          f"linear: shapes {tuple(x.shape)} and {tuple(weight.shape)} do not fit")
    _need(x.dtype is weight.dtype, f"linear: input is {x.dtype}, weight is {weight.dtype}")
    out_dtype = out_dtype or x.dtype
    _need(softcap is None or out_dtype is torch.float32, "linear: the soft-cap is applied to float32 results")
    if x.dtype is torch.float32:
        _need(out_dtype is torch.float32, "linear: the 32-bit path writes float32")
        _dense(x, "x"); _dense(weight, "weight")
        out = torch.empty((x.shape[0], weight.shape[0]), dtype=torch.float32, device=x.device)
        library.check(library.load().rdl_gemm_f32(_ptr(out), _ptr(x), _ptr(weight), x.shape[0], weight.shape[0],
                                                  x.shape[1], _stream(x)))
    elif _own_bf16_kernel(x, weight):
        return _gemm_bf16(x, weight, weight.shape[0], out_dtype, False, 0, softcap, status)
    else:
        _need(x.is_cuda, "kernels run on CUDA tensors only; there is no CPU path")
        out = torch.mm(x, weight.t(), out_dtype=torch.float32) if out_dtype is torch.float32 else torch.mm(x, weight.t())
    if softcap is not None:
        softcap_(out, softcap)
    return out


def linear_gated(x, weight_gate_up: torch.Tensor, activation: str, status: Optional[torch.Tensor] = None):
    """act(x Wg^T) * (x Wu^T) for the row-concatenated matrix [Wg; Wu] ([2I, in]) -> [rows, I].
    In bfloat16 this is one kernel (the activation is the product's epilogue); otherwise a product
    and the gated activation kernel."""
    _need(activation in ACTIVATIONS, f"unknown activation '{activation}', known: {sorted(ACTIVATIONS)}")
    _need(weight_gate_up.shape[0] % 2 == 0, "linear_gated: the weight must hold gate rows and as many up rows")
    if isinstance(x, DeferredRows):
        out = _linear_deferred(x, weight_gate_up, weight_gate_up.shape[0] // 2, x.dtype, True, ACTIVATIONS[activation], None, status)
        if out is not None:
            return out
        x = x.materialise()
    if _own_bf16_kernel(x, weight_gate_up):
        return _gemm_bf16(x, weight_gate_up, weight_gate_up.shape[0] // 2, x.dtype, True, ACTIVATIONS[activation], None, status)
    return gated_activation(linear(x, weight_gate_up), activation)


# ------------------------------------------------------------------------------------------
# position encoding, cache write, attention
# ------------------------------------------------------------------------------------------

class KVPages(NamedTuple):
    """One schedule entry's key/value storage and the page lists of the step's sequences."""
    k: torch.Tensor            # [pages, kv_heads, page_size, head_dim]
    v: torch.Tensor
    tables: torch.Tensor       # int32 [n_seqs, table_width]
    page_size: int
    ring_pages: int            # entries of a page list used as a ring (= table width when all keys are kept)


def rope_cache(qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, *, tok_seq, tok_pos,
               cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None, rotary_dim: int = 0,
               pages: Optional[KVPages] = None, seq_end: Optional[torch.Tensor] = None):
    """In place on packed rows [tokens, (n_heads + 2 n_kv_heads) * head_dim]: rotate query and key heads by
    the tables (if given), then write key and value rows to the cache (if `pages` is given)."""
    _dense(qkv, "qkv")
    T = qkv.shape[0]
    _need(qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim, "qkv width does not match the head counts")
    _int32(tok_pos, "tok_pos", T)
    _int32(tok_seq, "tok_seq", T)
    do_rope = cos is not None
    if do_rope:
        _need(cos.dtype is torch.float32 and sin.dtype is torch.float32 and cos.is_contiguous() and sin.is_contiguous()
              and cos.shape == sin.shape and cos.shape[1] * 2 == rotary_dim, "rotary tables must be float32 [positions, rotary_dim/2]")
    do_write = pages is not None and n_kv_heads > 0
    if do_write:
        _need(pages.k.dtype is qkv.dtype and pages.v.dtype is qkv.dtype, "cache dtype differs from the activations'")
        _need(tuple(pages.k.shape[1:]) == (n_kv_heads, pages.page_size, head_dim) and pages.k.is_contiguous()
              and pages.v.is_contiguous() and pages.v.shape == pages.k.shape, "cache storage has the wrong shape")
        _int32(pages.tables, "page tables")
        _int32(seq_end, "seq_end")
    library.check(library.load().rdl_rope_cache(
        _ptr(qkv), _dtype_code(qkv), T, n_heads, n_kv_heads, head_dim, rotary_dim,
        _ptr(cos), _ptr(sin), _ptr(tok_seq), _ptr(tok_pos), int(do_rope), int(do_write),
        _ptr(pages.k) if do_write else None, _ptr(pages.v) if do_write else None,
        _ptr(pages.tables) if do_write else None, pages.tables.shape[1] if do_write else 0,
        pages.page_size if do_write else 0, pages.ring_pages if do_write else 0,
        _ptr(seq_end) if do_write else None, _stream(qkv)))
    return qkv


PREFILL_QUERY_TILE = 64    # query rows of a tile in the lists the prefill attention kernels take


class AttentionBatch(NamedTuple):
    """The step's sequences as the attention kernels see them (device int32 tensors)."""
    n_tokens: int
    n_seqs: int
    tok_seq: torch.Tensor      # [tokens]
    tok_pos: torch.Tensor      # [tokens], -1 marks a padding row
    seq_start: torch.Tensor    # [seqs + 1]
    seq_past: torch.Tensor     # [seqs]
    seq_cached: torch.Tensor   # [seqs] keys below this position are read from the cache
    tile_seq: Optional[torch.Tensor] = None   # prefill: query tiles of PREFILL_QUERY_TILE rows
    tile_q0: Optional[torch.Tensor] = None
    n_tiles: int = 0
    max_keys: int = 0          # decode: longest key run any token of the batch reads (window applied)


def _attention_args(q, q_stride, k_new, v_new, kv_stride, out, b: AttentionBatch, pages: Optional[KVPages],
                    n_heads, n_kv_heads, head_dim, score_scale, softcap, window):
    a = AttentionArgs()
    a.dtype = _dtype_code(out)
    a.n_tokens, a.n_seqs = b.n_tokens, b.n_seqs
    a.n_heads, a.n_kv_heads, a.head_dim = n_heads, n_kv_heads, head_dim
    a.score_scale = float(score_scale)
    a.softcap = float(softcap or 0.0)
    a.window = int(window or 0)
    a.q, a.q_stride = q, q_stride
    a.k_new, a.v_new, a.kv_stride = k_new, v_new, kv_stride
    a.out, a.out_stride = out.data_ptr(), out.stride(0)
    a.tok_seq, a.tok_pos = b.tok_seq.data_ptr(), b.tok_pos.data_ptr()
    a.seq_start, a.seq_past, a.seq_cached = b.seq_start.data_ptr(), b.seq_past.data_ptr(), b.seq_cached.data_ptr()
    if pages is not None:
        a.k_cache, a.v_cache = pages.k.data_ptr(), pages.v.data_ptr()
        a.tables, a.table_width = pages.tables.data_ptr(), pages.tables.shape[1]
        a.page_size, a.ring_pages = pages.page_size, pages.ring_pages
    return a


@functools.lru_cache(maxsize=None)
def sm_count(device_index: int) -> int:
    return torch.cuda.get_device_properties(device_index).multi_processor_count


def choose_keys_per_split(n_tokens: int, n_kv_heads: int, max_keys: int, page_size: int, sms: int = 148) -> int:
    """Keys per block of the decode kernel: runs of four pages (a block then streams its pages one after
    the other, and fewer partial results are merged), shorter ones while that leaves the GPU with
    fewer than about one and a half blocks per multiprocessor (`sms` of them)."""
    blocks = lambda pages: n_tokens * n_kv_heads * ((max_keys + pages * page_size - 1) // (pages * page_size))
    for pages in (4, 2):
        if 2 * blocks(pages) >= 3 * sms:
            return pages * page_size
    return page_size


def attention(q: torch.Tensor, b: AttentionBatch, pages: Optional[KVPages], *, n_heads: int, n_kv_heads: int,
              head_dim: int, score_scale: float, softcap: Optional[float], window: Optional[int],
              new_kv: Optional[Tuple[torch.Tensor, int, int]] = None, kind: str = "auto",
              scratch=None, keys_per_split: Optional[int] = None, status: Optional[torch.Tensor] = None,
              rotate_and_write: Optional[Tuple[Optional[torch.Tensor], Optional[torch.Tensor], int]] = None):
    """Attention of the step's tokens over cache and new rows.

    q: [tokens, >= n_heads * head_dim] rows whose first n_heads * head_dim values are the (rotated)
    query heads; the row stride may be larger (packed q/k/v rows).
    new_kv: (rows, k_col, v_col) - this step's packed rows and the columns at which the rotated
    keys and the values start; needed when `b.seq_cached` says that new keys are not in the cache.
    kind: "plain" (float arithmetic, any dtype), "prefill" (bfloat16, mma.sync tensor cores, keys from
    cache and packed rows), "prefill_tc" (bfloat16, TMA + tcgen05, for sequences that start at position 0
    with head_dim a multiple of 64), "decode" (bfloat16, split keys; reads the cache only), or "auto".
    scratch: callable(nbytes) -> zero-initialised float32 tensor that only this kernel writes, for
    the decode kernel's counters and partial results.  status: int32 tensor that a kernel sets
    non-zero when it gives up on a bounded wait.
    rotate_and_write (kind "decode", one token per sequence, `b` describing all keys as cached):
    (cos, sin, rotary_dim) - q and new_kv are the rows as the projection left them; the kernel rotates
    the query and key heads by the float32 tables [positions, rotary_dim / 2] (None, None, 0: no
    rotation), writes the new key and value rows into the cache and attends over the cache including
    them.  The packed rows themselves stay as they are.
    Returns [tokens, n_heads * head_dim] in the dtype of q."""
    _need(q.dim() == 2 and q.stride(1) == 1 and q.shape[1] >= n_heads * head_dim, "attention: bad query rows")
    T = q.shape[0]
    _need(T >= b.n_tokens, "attention: fewer rows than tokens")
    out = torch.empty((T, n_heads * head_dim), dtype=q.dtype, device=q.device)
    es = q.element_size()
    k_new = v_new = None
    kv_stride = 0
    if new_kv is not None:
        rows, k_col, v_col = new_kv
        _need(rows.dtype is q.dtype and rows.dim() == 2 and rows.stride(1) == 1 and
              rows.shape[1] >= max(k_col, v_col) + n_kv_heads * head_dim, "attention: bad new key/value rows")
        k_new, v_new, kv_stride = rows.data_ptr() + k_col * es, rows.data_ptr() + v_col * es, rows.stride(0)
    a = _attention_args(q.data_ptr(), q.stride(0), k_new, v_new, kv_stride, out, b, pages, n_heads, n_kv_heads,
                        head_dim, score_scale, softcap, window)
    if pages is not None:
        _need(pages.k.dtype is q.dtype, "attention: cache dtype differs from the activations'")
    fast_ok = q.dtype is torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 256
    if kind == "auto":
        kind = "prefill" if fast_ok and b.n_tiles > 0 else "plain"
    lib = library.load()
    if kind == "plain":
        library.check(lib.rdl_attention_plain(ctypes.byref(a), _stream(q)))
    elif kind in ("prefill", "prefill_tc"):
        _need(b.tile_seq is not None and b.tile_q0 is not None, "attention: prefill needs query tiles")
        a.tile_seq, a.tile_q0, a.n_tiles = b.tile_seq.data_ptr(), b.tile_q0.data_ptr(), b.n_tiles
        if kind == "prefill_tc":
            # sequences that start at position 0, packed q/k/v rows, head_dim a multiple of 64
            _need(new_kv is not None and new_kv[0] is q, "attention: the tcgen05 prefill kernel reads packed q/k/v rows")
            a.status = _status(status)
            library.check(lib.rdl_attention_prefill_tc(ctypes.byref(a), q.stride(0), _stream(q)))
        else:
            library.check(lib.rdl_attention_prefill(ctypes.byref(a), _stream(q)))
    elif kind == "decode":
        _need(pages is not None, "attention: decode reads the cache")
        ks = keys_per_split or choose_keys_per_split(b.n_tokens, n_kv_heads, b.max_keys, pages.page_size,
                                                     sm_count(q.device.index or 0))
        a.keys_per_split = ks
        # a run of max_keys positions can straddle one more split than its length suggests
        a.max_splits = (max(b.max_keys, 1) + ks - 1) // ks + 1
        need = lib.rdl_attention_decode_scratch_bytes(b.n_tokens, n_heads, n_kv_heads, head_dim, a.max_splits)
        # the counters at the start of the scratch must be zero before a launch; the kernel leaves them so
        buf = scratch(need) if scratch is not None else torch.zeros(-(-need // 4), dtype=torch.float32, device=q.device)
        _need(buf.dtype is torch.float32 and buf.numel() * 4 >= need, "attention: decode scratch too small")
        a.scratch, a.scratch_bytes = buf.data_ptr(), buf.numel() * 4
        a.counter_bytes = lib.rdl_attention_decode_counter_bytes(b.n_tokens, n_kv_heads)
        a.status = _status(status)
        if rotate_and_write is not None:
            cos, sin, rotary_dim = rotate_and_write
            _need(new_kv is not None, "attention: rotate_and_write needs the step's key and value rows")
            if rotary_dim:
                _need(cos.dtype is torch.float32 and sin.dtype is torch.float32 and cos.is_contiguous() and sin.is_contiguous()
                      and cos.shape == sin.shape and cos.shape[1] * 2 == rotary_dim, "rotary tables must be float32 [positions, rotary_dim/2]")
                a.rope_cos, a.rope_sin = cos.data_ptr(), sin.data_ptr()
            a.rotary_dim, a.new_rows = int(rotary_dim), 1
        library.check(lib.rdl_attention_decode(ctypes.byref(a), _stream(q)))
    else:
        raise KernelError(f"attention: unknown kind '{kind}'")
    return out


# ------------------------------------------------------------------------------------------
# random weights
# ------------------------------------------------------------------------------------------

def random_normal(shape, key: int, std: float, dtype: torch.dtype, device) -> torch.Tensor:
    """N(0, std) values of the tensor with 64-bit `key`, made on the device: element j depends only on
    (key, j) and equals, bit for bit in float32, what `weights.counter_random.normal` makes on the host."""
    out = torch.empty(shape, dtype=dtype, device=device)
    library.check(library.load().rdl_random_normal(_ptr(out), _dtype_code(out), out.numel(), int(key) & (2**64 - 1),
                                                   float(std), _stream(out)))
    return out


# ------------------------------------------------------------------------------------------
# sampling
# ------------------------------------------------------------------------------------------

def sample(logits: torch.Tensor, *, temperature: float, top_k: Optional[int] = None, top_p: Optional[float] = None,
           repetition_penalty: Optional[float] = None, seed: int = 0, row_stream: Optional[torch.Tensor] = None,
           row_step: Optional[torch.Tensor] = None, history: Optional[torch.Tensor] = None,
           history_start: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
           host_out: Optional[torch.Tensor] = None):
    """One token per row of float32 logits [rows, vocab] -> int32 [rows].  host_out: pinned int32 host memory of
    at least `rows` values that the kernel writes the tokens to as well (readable once the kernel has ended)."""
    _need(logits.dtype is torch.float32 and logits.dim() == 2 and logits.is_contiguous(),
          "sample takes contiguous float32 logits [rows, vocab]")
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    prm = SamplingArgs(float(temperature), int(top_k or 0), float(top_p if top_p is not None else 1.0),
                       float(repetition_penalty if repetition_penalty is not None else 1.0), int(seed) & (2**64 - 1))
    work = None
    if temperature >= 1e-7:
        work = torch.empty_like(logits)
        if row_stream is not None:
            _need(row_stream.dtype is torch.int64 and row_stream.numel() >= rows, "row_stream must be int64 [rows]")
        if row_step is not None:
            _int32(row_step, "row_step", rows)
        if history is not None:
            _int32(history, "history")
            _int32(history_start, "history_start", rows + 1)
    if host_out is not None:
        _need(host_out.dtype is torch.int32 and host_out.is_pinned() and host_out.is_contiguous() and host_out.numel() >= rows,
              "sample: host_out must be pinned int32 host memory with a value per row")
    library.check(library.load().rdl_sample(_ptr(out), host_out.data_ptr() if host_out is not None else None, _ptr(logits), rows, vocab,
                                            ctypes.byref(prm), _ptr(row_stream),
                                            _ptr(row_step), _ptr(history), _ptr(history_start), _ptr(work), _stream(logits)))
    return out


def upload_batch(dst: torch.Tensor, src_pinned: torch.Tensor, n_ints: int, fed: Optional[Tuple[torch.Tensor, int, int, int]] = None):
    """A step's int32 batch description from pinned host memory to the device by a kernel (no copy engine between the
    kernels of two steps).  fed = (sampled ids on the device, where the description lists their rows, where its
    tokens lie, how many): those tokens are taken from `sampled` on the way."""
    _need(dst.dtype is torch.int32 and dst.is_cuda and src_pinned.dtype is torch.int32 and src_pinned.is_pinned()
          and dst.numel() >= n_ints and src_pinned.numel() >= n_ints, "upload_batch: int32 device buffer and pinned int32 host buffer")
    sampled, src_at, tok_at, n_fed = fed if fed is not None else (None, 0, 0, 0)
    if sampled is not None:
        _int32(sampled, "sampled")
    library.check(library.load().rdl_upload_batch(_ptr(dst), src_pinned.data_ptr(), n_ints, _ptr(sampled), src_at, tok_at, n_fed,
                                                  _stream(dst)))
