"""Each CUDA kernel alone against its plain reference (tests/kernel_refs.py, float64), at sizes
other than the engine's: odd row counts, head sizes in steps of 16, widths and vocabularies that
are no power of two, windows shorter and longer than the context, ring caches that wrap.
Outputs are allocated by the kernels' wrappers with torch.empty, so stale values would show."""
import math

import numpy as np
import pytest
import torch

import kernel_refs as ref
from rust_deeplearning_b200.kernels import ops
from rust_deeplearning_b200.sampling.sampler import uniform_for

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
BF16_EPS = 2.0 ** -8      # half a unit in the last place of bfloat16, relative


def rnd(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(DEV)


def assert_close(got, want, dtype, rel=4.0, what="", f32_tol=2e-5):
    """float32 results agree to ~1e-5 relative to the tensor's scale; bfloat16 results to a few
    units of bfloat16 rounding of that scale.  Products that sum thousands of terms in float32 pass
    f32_tol = 1e-4: 2048 terms x 2^-24 per addition bounds the sum's rounding at 1.2e-4 of its scale."""
    got, want = got.double().cpu(), want.double().cpu()
    assert got.shape == want.shape, (got.shape, want.shape)
    assert torch.isfinite(got).all(), f"{what}: non-finite output"
    scale = max(want.abs().max().item(), 1e-6)
    tol = (f32_tol if dtype is torch.float32 else rel * BF16_EPS) * scale
    err = (got - want).abs().max().item()
    assert err <= tol, f"{what}: max error {err:.3e} > {tol:.3e} (scale {scale:.3e})"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_rows(dtype):
    table = rnd((131, 80), dtype, 0)
    ids = torch.tensor([0, 130, 5, 5, 77], dtype=torch.int32, device=DEV)
    got = ops.embed_rows(table, ids, math.sqrt(80))
    assert_close(got, ref.embed_rows(table, ids, math.sqrt(80)), torch.float32)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    bad = ops.embed_rows(table, torch.tensor([3, 131], dtype=torch.int32, device=DEV), 1.0, status)
    assert status.item() == 1 and torch.isnan(bad[1]).all() and torch.isfinite(bad[0]).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [80, 131, 2304, 5000, 10000])
def test_norm_residual_norm(dtype, hidden):
    rows = 7
    x = rnd((rows, hidden), dtype, 1, 3.0)
    w1 = ops.NormParams(rnd((hidden,), dtype, 2, 0.5), 1e-5, 1.0)
    w2 = ops.NormParams(rnd((hidden,), torch.float32, 3, 0.5), 1e-6, 0.0)   # a norm weight kept in 32 bits
    res = rnd((rows, hidden), torch.float32, 4, 2.0)
    # norm only
    assert_close(ops.norm_residual_norm(x, second=w1), ref.norm_residual_norm(x, second=w1), dtype, what="norm")
    # post-norm, residual add, pre-norm in one kernel
    r_got, r_ref = res.clone(), res.clone()
    y = ops.norm_residual_norm(x, first=w1, residual=r_got, second=w2, out_dtype=dtype)
    y_ref = ref.norm_residual_norm(x, first=w1, residual=r_ref, second=w2, out_dtype=dtype)
    assert_close(r_got, r_ref, torch.float32, what="residual")
    assert_close(y, y_ref, dtype, what="fused output")
    # residual update without output, and a plain add
    r_got, r_ref = res.clone(), res.clone()
    assert ops.norm_residual_norm(x, first=None, residual=r_got, want_output=False) is None
    ref.norm_residual_norm(x, first=None, residual=r_ref, want_output=False)
    assert_close(r_got, r_ref, torch.float32, what="plain add")
    # gathered rows
    idx = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    assert_close(ops.norm_residual_norm(res, second=w2, out_dtype=dtype, row_index=idx),
                 ref.norm_residual_norm(res, second=w2, out_dtype=dtype, row_index=idx), dtype, what="gathered")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_activation_softcap_add_convert(dtype):
    gu = rnd((5, 2 * 112), dtype, 5, 2.0)
    for act in ("gelu_pytorch_tanh", "silu"):
        assert_close(ops.gated_activation(gu, act), ref.gated_activation(gu, act), dtype, what=act)
    z = rnd((3, 131), torch.float32, 6, 40.0)
    assert_close(ops.softcap_(z.clone(), 30.0), ref.softcap_(z.clone(), 30.0), torch.float32, what="softcap")
    res = rnd((5, 112), torch.float32, 7)
    x = rnd((5, 112), dtype, 8)
    assert_close(ops.residual_add_(res.clone(), x), ref.residual_add_(res.clone(), x), torch.float32, what="add")
    idx = torch.tensor([4, 4, 1], dtype=torch.int32, device=DEV)
    assert_close(ops.convert_rows(res, dtype, idx), ref.convert_rows(res, dtype, idx), dtype, what="convert")


@pytest.mark.parametrize("m,n,k", [(1, 131, 80), (7, 300, 257), (129, 65, 64), (64, 64, 16)])
def test_gemm_f32_is_exact_float32(m, n, k):
    x, w = rnd((m, k), torch.float32, 9), rnd((n, k), torch.float32, 10)
    got = ops.linear(x, w)
    assert_close(got, ref.linear(x, w), torch.float32, what="gemm_f32")
    # a row's result does not depend on the other rows of the batch: bit-equal
    alone = ops.linear(x[m // 2:m // 2 + 1].contiguous(), w)
    assert torch.equal(alone[0], got[m // 2])


def test_linear_bf16_float32_output():
    x, w = rnd((5, 96), torch.bfloat16, 11), rnd((384, 96), torch.bfloat16, 12)
    assert ops.linear(x, w, out_dtype=torch.float32).dtype is torch.float32
    assert_close(ops.linear(x, w, out_dtype=torch.float32), ref.linear(x, w, torch.float32), torch.float32, what="head")
    assert_close(ops.linear(x, w), ref.linear(x, w), torch.bfloat16, what="linear")


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("n,k", [(131, 80), (384, 96), (2304, 2048), (40, 1160), (16, 8)])
def test_skinny_gemm(m, n, k):
    """The weight-streaming kernel for few rows: plain, float32 output with soft-cap, and gated."""
    x, w = rnd((m, k), torch.bfloat16, 13), rnd((n, k), torch.bfloat16, 14, 0.2)
    assert ops._skinny_ok(x, w)
    assert_close(ops.linear(x, w), ref.linear(x, w), torch.bfloat16, what="plain")
    assert_close(ops.linear(x, w, out_dtype=torch.float32), ref.linear(x, w, torch.float32), torch.float32, what="float32 out")
    assert_close(ops.linear(x, w, out_dtype=torch.float32, softcap=3.0), ref.linear(x, w, torch.float32, softcap=3.0),
                 torch.float32, what="soft-cap")
    wgu = rnd((2 * n, k), torch.bfloat16, 15, 0.2)
    for act in ("gelu_pytorch_tanh", "silu"):
        assert_close(ops.linear_gated(x, wgu, act), ref.linear_gated(x, wgu, act), torch.bfloat16, what=f"gated {act}")
    # the library product and the activation kernel (the route of operands the own kernels do not take) give the same
    x17 = rnd((17, k), torch.bfloat16, 16)
    assert not ops._own_bf16_kernel(x17, w)
    assert_close(ops.linear_gated(x17, wgu, "silu"), ref.linear_gated(x17, wgu, "silu"), torch.bfloat16, what="17 rows")
    assert_close(ops.gated_activation(torch.mm(x17, wgu.t()), "gelu_pytorch_tanh"), ref.linear_gated(x17, wgu, "gelu_pytorch_tanh"),
                 torch.bfloat16, what="gated, library product")


@pytest.mark.parametrize("m,n,k", [(8, 2304, 9216), (5, 100, 7000), (1, 16, 6152), (7, 2368, 3080)])
def test_skinny_gemm_long_rows(m, n, k):
    """Rows of many tiles: a narrow output has one block a multiprocessor with the longer ring, which goes
    round more than once within a unit (9216 = 9 tiles of 1024 through 6 places); 7000 and 6152 end in a
    short tile; 2368 outputs are 148 units, the most that still get the longer ring."""
    x, w = rnd((m, k), torch.bfloat16, 43), rnd((n, k), torch.bfloat16, 44, 0.2)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert ops._skinny_ok(x, w)
    assert_close(ops.linear(x, w, status=status), ref.linear(x, w), torch.bfloat16, what="plain")
    assert_close(ops.linear(x, w, out_dtype=torch.float32, status=status), ref.linear(x, w, torch.float32), torch.float32,
                 what="float32 out", f32_tol=k * 2.0 ** -24)
    if n % 2 == 0:
        assert_close(ops.linear_gated(x, w, "gelu_pytorch_tanh", status=status), ref.linear_gated(x, w, "gelu_pytorch_tanh"),
                     torch.bfloat16, what="gated")
    assert status.item() == 0


@pytest.mark.parametrize("m", [2, 8, 13])
def test_skinny_gemm_with_more_units_than_blocks_fit(m):
    """A wide output has more 16-row units than blocks fit the GPU at once: blocks then go on to further
    units (a few thousand here, with a tail that does not fill the last unit), in every form."""
    n, k = 40003, 264
    x, w = rnd((m, k), torch.bfloat16, 33), rnd((n, k), torch.bfloat16, 34, 0.2)
    # the reference forms [m, n, k] in float64: in pieces of the output
    got = ops.linear(x, w, out_dtype=torch.float32, softcap=2.0)
    for lo in range(0, n, 8192):
        assert_close(got[:, lo:lo + 8192], ref.linear(x, w[lo:lo + 8192], torch.float32, softcap=2.0), torch.float32, what=f"columns from {lo}")
    n2 = 9001
    wgu = rnd((2 * n2, k), torch.bfloat16, 35, 0.2)
    assert_close(ops.linear_gated(x, wgu, "gelu_pytorch_tanh"), ref.linear_gated(x, wgu, "gelu_pytorch_tanh"), torch.bfloat16, what="gated")
    assert_close(ops.linear(x, w[:n2]), ref.linear(x, w[:n2]), torch.bfloat16, what="plain")


@pytest.mark.parametrize("m", [1, 3, 8])
@pytest.mark.parametrize("width,k_in,n_out", [(2304, 2048, 4096), (80, 96, 131), (1000, 264, 20003), (3584, 512, 600)])
def test_deferred_norms_around_few_row_products(m, width, k_in, n_out):
    """norm(branch) + stream, norm of the sum, next product - with the two norms split between the epilogue of the
    product before and the product after (no kernel of their own): the product's result, the updated stream
    and the next operand's first half against the float64 formulas; a second product on the same rows, a
    selection of rows, and the same rows made into a tensor."""
    x, w_p = rnd((m, k_in), torch.bfloat16, 70), rnd((width, k_in), torch.bfloat16, 71, 0.2)
    h = rnd((m, width), torch.float32, 72, 2.0)
    post = ops.NormParams(rnd((width,), torch.bfloat16, 73, 0.5), 1e-5, 1.0)
    then = ops.NormParams(rnd((width,), torch.float32, 74, 0.5), 1e-6, 0.0)       # a norm weight kept in 32 bits
    nxt = ops.NormParams(rnd((width,), torch.bfloat16, 75, 0.5), 1e-6, 1.0)
    w_c = rnd((n_out, width), torch.bfloat16, 76, 0.2)
    w_gu = rnd((2 * 72, width), torch.bfloat16, 77, 0.2)
    # float64
    y = x.double() @ w_p.double().t()
    h_new = h.double() + ref._rms(y, post)
    xn = ref._rms(h_new, then)
    z = xn @ w_c.double().t()
    # split form
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    operand = ops.scaled_rows(h, then)
    assert_close(operand[:m], h.double() * (then.weight.double() + then.offset), torch.bfloat16, rel=1.0, what="first half of the operand")
    br = ops.linear_branch(x, w_p, ops.BranchSink(h, post, then, operand), status=status)
    assert isinstance(br, ops.Branch)
    h_out, next_operand = torch.empty_like(h), torch.empty_like(operand)
    d = ops.DeferredRows(br, h_out, nxt, next_operand)
    got = ops.linear(d, w_c, status=status)
    assert d.consumed and got.dtype is torch.bfloat16
    assert_close(got, z, torch.bfloat16, what="product after the norms")
    assert_close(h_out, h_new, torch.bfloat16, rel=1.0, what="updated stream")       # the branch is rounded to bfloat16 before the sum, as in the one-kernel form
    assert_close(next_operand[:m], h_new * (nxt.weight.double() + nxt.offset), torch.bfloat16, rel=1.5, what="next operand")
    # the former route, for the record: a product, the fused norm kernel, a product
    res = h.clone()
    old = ops.linear(ops.norm_residual_norm(ops.linear(x, w_p), first=post, residual=res, second=then, out_dtype=torch.bfloat16), w_c)
    scale = z.abs().max().item()
    print(f"[deferred norms] m={m} width={width}: error / scale split {(got.double().cpu() - z.cpu()).abs().max().item() / scale:.2e}, "
          f"separate kernels {(old.double().cpu() - z.cpu()).abs().max().item() / scale:.2e}")
    # a second product on the same rows (gated, float32 output with soft-cap), then a selection of rows
    assert_close(ops.linear_gated(d, w_gu, "gelu_pytorch_tanh", status=status),
                 ref.gated_activation(xn @ w_gu.double().t(), "gelu_pytorch_tanh"), torch.bfloat16, what="gated")
    assert_close(ops.linear(d, w_c, out_dtype=torch.float32, softcap=3.0, status=status), 3.0 * torch.tanh(z / 3.0),
                 torch.bfloat16, what="float32 with soft-cap")
    rows = torch.tensor([m - 1, 0], dtype=torch.int32, device=DEV)
    h_out2 = torch.empty_like(h)
    d2 = ops.DeferredRows(br, h_out2, row_index=rows)
    assert_close(ops.linear(d2, w_c, status=status), z[rows.long()], torch.bfloat16, what="selected rows")
    assert torch.equal(h_out2, h_out)
    # the same rows as a tensor (a consumer that cannot take the split form)
    h_out3, next3 = torch.empty_like(h), torch.empty_like(operand)
    d3 = ops.DeferredRows(br, h_out3, nxt, next3)
    assert_close(d3.materialise(), xn, torch.bfloat16, what="materialised")
    assert_close(h_out3, h_new, torch.bfloat16, rel=1.0, what="updated stream, materialised")
    assert_close(next3[:m], h_new * (nxt.weight.double() + nxt.offset), torch.bfloat16, rel=1.5, what="next operand, materialised")
    # a weight the streaming kernel does not take (a view that starts off a 16-byte boundary): the rows are made into a tensor
    w_odd = torch.empty(n_out * width + 1, dtype=torch.bfloat16, device=DEV)[1:].view(n_out, width).copy_(w_c)
    d4 = ops.DeferredRows(br, torch.empty_like(h), nxt, torch.empty_like(operand))
    assert_close(ops.linear(d4, w_odd), z, torch.bfloat16, what="library product after materialising")
    assert status.item() == 0


@pytest.mark.parametrize("m", [128, 129, 200, 2048])
@pytest.mark.parametrize("n,k", [(256, 64), (384, 96), (131, 80), (2304, 2048), (520, 1160)])
def test_tcgen05_gemm(m, n, k):
    """The TMA + tcgen05 kernel for many rows: tiles, tails in every dimension, all epilogues."""
    x, w = rnd((m, k), torch.bfloat16, 17), rnd((n, k), torch.bfloat16, 18, 0.2)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert ops.PREFILL_GEMM == "tcgen05" and ops._own_bf16_kernel(x, w) and not ops._skinny_ok(x, w)
    assert_close(ops.linear(x, w, status=status), ref.linear(x, w), torch.bfloat16, what="plain")
    assert_close(ops.linear(x, w, out_dtype=torch.float32, softcap=3.0, status=status), ref.linear(x, w, torch.float32, softcap=3.0),
                 torch.float32, what="float32 out, soft-cap", f32_tol=1e-4)
    wgu = rnd((2 * n, k), torch.bfloat16, 19, 0.2)
    for act in ("gelu_pytorch_tanh", "silu"):
        assert_close(ops.linear_gated(x, wgu, act, status=status), ref.linear_gated(x, wgu, act), torch.bfloat16, what=f"gated {act}")
    assert status.item() == 0


@pytest.mark.parametrize("m,n,k", [(300, 520, 4160), (129, 256, 4096), (513, 131, 4104)])
def test_tcgen05_gemm_pair_long_sum(m, n, k):
    """Sums of 4096 terms and more with more than one tile of rows go to the kernel that puts two
    multiprocessors on one tile (as the gated products above do): tails in every dimension."""
    x, w = rnd((m, k), torch.bfloat16, 27), rnd((n, k), torch.bfloat16, 28, 0.2)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert_close(ops.linear(x, w, status=status), ref.linear(x, w), torch.bfloat16, what="plain")
    # float accumulation over k terms: k x 2^-24 bounds the sum's rounding relative to its scale
    assert_close(ops.linear(x, w, out_dtype=torch.float32, status=status), ref.linear(x, w, torch.float32), torch.float32,
                 what="float32 out", f32_tol=k * 2.0 ** -24)
    assert status.item() == 0


# ------------------------------------------------------------------------------------------
# position encoding, cache write and attention
# ------------------------------------------------------------------------------------------

class Case:
    """A packed batch over a paged cache, built on the host like the engine builds it."""

    def __init__(self, *, past, new, n_heads, n_kv_heads, head_dim, page_size, window, dtype, seed,
                 shuffle_pages=True, max_context=None):
        from rust_deeplearning_b200.cache.cache import ring_pages_for
        self.n_heads, self.n_kv_heads, self.head_dim, self.window, self.dtype = n_heads, n_kv_heads, head_dim, window, dtype
        self.page_size = page_size
        n = len(past)
        totals = [p + s for p, s in zip(past, new)]
        max_context = max_context or max(totals)
        ctx_pages = -(-max_context // page_size)
        ring = ring_pages_for(window, page_size) if window else ctx_pages
        self.ring_pages = min(ring, ctx_pages)
        rng = np.random.default_rng(seed)
        n_pages = n * self.ring_pages + 3
        order = rng.permutation(n_pages) if shuffle_pages else np.arange(n_pages)
        tables = np.zeros((n, self.ring_pages), dtype=np.int32)
        for i in range(n):
            tables[i] = order[i * self.ring_pages:(i + 1) * self.ring_pages]
        T = sum(new)
        tok_seq = np.concatenate([np.full(s, i) for i, s in enumerate(new)]).astype(np.int32)
        tok_pos = np.concatenate([np.arange(p, p + s) for p, s in zip(past, new)]).astype(np.int32)
        starts = np.concatenate([[0], np.cumsum(new)]).astype(np.int32)
        tiles = [(i, q0) for i, s in enumerate(new) for q0 in range(0, s, 64)]
        dev = lambda a: torch.from_numpy(np.asarray(a, dtype=np.int32)).to(DEV)
        self.T, self.n = T, n
        self.tok_seq, self.tok_pos, self.seq_start = dev(tok_seq), dev(tok_pos), dev(starts)
        self.seq_past, self.seq_end = dev(past), dev(totals)
        self.tile_seq, self.tile_q0 = dev([t[0] for t in tiles]), dev([t[1] for t in tiles])
        self.n_tiles = len(tiles)
        self.max_total = max(totals)
        self.k = rnd((n_pages, n_kv_heads, page_size, head_dim), dtype, seed + 1)
        self.v = rnd((n_pages, n_kv_heads, page_size, head_dim), dtype, seed + 2)
        self.pages = ops.KVPages(self.k, self.v, dev(tables), page_size, self.ring_pages)
        width = (n_heads + 2 * n_kv_heads) * head_dim
        self.qkv = rnd((T, width), dtype, seed + 3)

    def batch(self, keys_in_cache):
        cached = self.seq_past if keys_in_cache == "past" else self.seq_end
        max_keys = min(self.max_total, self.window) if self.window else self.max_total
        return ops.AttentionBatch(self.T, self.n, self.tok_seq, self.tok_pos, self.seq_start, self.seq_past, cached,
                                  self.tile_seq, self.tile_q0, self.n_tiles, max_keys)

    def kw(self, scale=None, softcap=None):
        return dict(n_heads=self.n_heads, n_kv_heads=self.n_kv_heads, head_dim=self.head_dim,
                    score_scale=scale or 1.0 / math.sqrt(self.head_dim), softcap=softcap, window=self.window)

    def new_kv(self):
        q = self.n_heads * self.head_dim
        return (self.qkv, q, q + self.n_kv_heads * self.head_dim)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("head_dim,rotary", [(16, 16), (48, 32), (256, 256)])
def test_rope_and_cache_write(dtype, head_dim, rotary):
    c = Case(past=[0, 5, 30], new=[7, 1, 40], n_heads=3, n_kv_heads=1, head_dim=head_dim, page_size=4,
             window=8, dtype=dtype, seed=20)           # ring of 4 pages = 16 rows, wrapped by the third sequence
    half = rotary // 2
    ang = torch.arange(100, dtype=torch.float64)[:, None] / (50.0 ** (torch.arange(half, dtype=torch.float64) / half))
    cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)
    q_got, q_ref = c.qkv.clone(), c.qkv.clone()
    k_ref, v_ref = c.k.clone(), c.v.clone()
    pages_ref = ops.KVPages(k_ref, v_ref, c.pages.tables, c.page_size, c.ring_pages)
    ops.rope_cache(q_got, 3, 1, head_dim, tok_seq=c.tok_seq, tok_pos=c.tok_pos, cos=cos, sin=sin, rotary_dim=rotary,
                   pages=c.pages, seq_end=c.seq_end)
    ref.rope_cache(q_ref, 3, 1, head_dim, tok_seq=c.tok_seq, tok_pos=c.tok_pos, cos=cos, sin=sin, rotary_dim=rotary,
                   pages=pages_ref, seq_end=c.seq_end)
    assert_close(q_got, q_ref, dtype, rel=1.0, what="rotated rows")
    assert_close(c.k, k_ref, dtype, rel=1.0, what="key cache")
    assert_close(c.v, v_ref, dtype, rel=1.0, what="value cache")


ATTN_SHAPES = [
    # past, new, heads, kv heads, head_dim, page, window
    dict(past=[0], new=[1], n_heads=1, n_kv_heads=1, head_dim=16, page_size=64, window=None),
    dict(past=[0, 0, 0], new=[5, 129, 70], n_heads=4, n_kv_heads=2, head_dim=32, page_size=16, window=None),
    dict(past=[0, 0], new=[200, 33], n_heads=6, n_kv_heads=1, head_dim=48, page_size=8, window=24),
    dict(past=[90, 3, 0], new=[70, 130, 1], n_heads=2, n_kv_heads=2, head_dim=80, page_size=16, window=50),
    dict(past=[10, 0], new=[65, 64], n_heads=8, n_kv_heads=4, head_dim=256, page_size=64, window=None),
    dict(past=[0], new=[150], n_heads=3, n_kv_heads=3, head_dim=128, page_size=32, window=100),
]


@pytest.mark.parametrize("shape", ATTN_SHAPES)
@pytest.mark.parametrize("dtype,kind", [(torch.float32, "plain"), (torch.bfloat16, "plain"), (torch.bfloat16, "prefill")])
def test_attention_over_cache_and_new_rows(shape, dtype, kind):
    c = Case(dtype=dtype, seed=30, **shape)
    b = c.batch("past")
    for softcap in (None, 5.0):
        got = ops.attention(c.qkv, b, c.pages, new_kv=c.new_kv(), kind=kind, **c.kw(softcap=softcap))
        want = ref.attention(c.qkv, b, c.pages, new_kv=c.new_kv(), **c.kw(softcap=softcap))
        assert_close(got, want, dtype, rel=6.0, what=f"{kind} softcap={softcap}")


TC_SHAPES = [
    dict(new=[1], n_heads=1, n_kv_heads=1, head_dim=64, window=None),
    dict(new=[5, 129, 70], n_heads=4, n_kv_heads=2, head_dim=64, window=None),
    dict(new=[300, 33, 128], n_heads=6, n_kv_heads=1, head_dim=128, window=100),
    dict(new=[257, 64], n_heads=8, n_kv_heads=4, head_dim=256, window=None),
    dict(new=[700], n_heads=2, n_kv_heads=2, head_dim=256, window=130),
    dict(new=[130, 1, 260], n_heads=3, n_kv_heads=3, head_dim=192, window=64),
]


@pytest.mark.parametrize("shape", TC_SHAPES)
def test_tcgen05_prefill_attention(shape):
    """The TMA + tcgen05 prefill kernel (prompts that start at position 0) against the plain reference."""
    shape = dict(shape)
    new = shape.pop("new")
    c = Case(past=[0] * len(new), new=new, dtype=torch.bfloat16, seed=35, page_size=64, **shape)
    b = c.batch("past")
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for softcap in (None, 5.0):
        got = ops.attention(c.qkv, b, c.pages, new_kv=c.new_kv(), kind="prefill_tc", status=status, **c.kw(softcap=softcap))
        want = ref.attention(c.qkv, b, c.pages, new_kv=c.new_kv(), **c.kw(softcap=softcap))
        assert status.item() == 0
        assert_close(got, want, torch.bfloat16, rel=6.0, what=f"tcgen05 prefill softcap={softcap}")


DECODE_SHAPES = [
    dict(past=[0, 63, 64, 700], n_heads=8, n_kv_heads=4, head_dim=256, page_size=64, window=None),
    dict(past=[5, 1000, 300], n_heads=6, n_kv_heads=1, head_dim=32, page_size=16, window=None),
    dict(past=[2000, 17, 130], n_heads=4, n_kv_heads=2, head_dim=128, page_size=64, window=100),
    dict(past=[511, 512], n_heads=3, n_kv_heads=3, head_dim=48, page_size=32, window=512),
    dict(past=[77], n_heads=16, n_kv_heads=2, head_dim=80, page_size=64, window=33),
    dict(past=[300, 9], n_heads=5, n_kv_heads=1, head_dim=64, page_size=48, window=None),
]


@pytest.mark.parametrize("shape", DECODE_SHAPES)
@pytest.mark.parametrize("keys_per_split", [None, "one_page", "eight_pages"])
def test_decode_attention_over_cache(shape, keys_per_split):
    shape = dict(shape)
    past = shape.pop("past")
    c = Case(past=past, new=[1] * len(past), dtype=torch.bfloat16, seed=40, **shape)
    b = c.batch("all")
    ks = {None: None, "one_page": c.page_size, "eight_pages": 8 * c.page_size}[keys_per_split]
    for softcap in (None, 7.0):
        got = ops.attention(c.qkv, b, c.pages, kind="decode", keys_per_split=ks, **c.kw(softcap=softcap))
        want = ref.attention(c.qkv, b, c.pages, **c.kw(softcap=softcap))
        assert_close(got, want, torch.bfloat16, rel=6.0, what=f"decode softcap={softcap}")
        plain = ops.attention(c.qkv, b, c.pages, kind="plain", **c.kw(softcap=softcap))
        assert_close(plain, want, torch.bfloat16, rel=6.0, what="plain on the same case")


@pytest.mark.parametrize("shape", DECODE_SHAPES)
@pytest.mark.parametrize("rotary", ["whole", "half", "none"])
def test_decode_attention_rotates_and_writes_the_new_rows(shape, rotary):
    """The decode kernel doing the rotation and the cache write itself: output, both caches and the
    untouched packed rows against the rotation + cache write + attention of the reference."""
    shape = dict(shape)
    past = shape.pop("past")
    c = Case(past=past, new=[1] * len(past), dtype=torch.bfloat16, seed=45, **shape)
    hd = c.head_dim
    rotary_dim = {"whole": hd, "half": hd // 2, "none": 0}[rotary]
    if rotary_dim % 16:
        pytest.skip("the kernel takes rotations over a multiple of 16 elements")
    b = c.batch("all")
    half = max(rotary_dim // 2, 1)
    ang = torch.arange(max(past) + 2, dtype=torch.float64)[:, None] / (50.0 ** (torch.arange(half, dtype=torch.float64) / half))
    cos, sin = ang.cos().float().to(DEV).contiguous(), ang.sin().float().to(DEV).contiguous()
    rw = (cos, sin, rotary_dim) if rotary_dim else (None, None, 0)
    ref_pages = ops.KVPages(c.k.clone(), c.v.clone(), c.pages.tables, c.page_size, c.ring_pages)
    want = ref.attention(c.qkv, b, ref_pages, new_kv=c.new_kv(), rotate_and_write=rw, **c.kw(softcap=9.0))
    rows_before = c.qkv.clone()
    for ks in (None, c.page_size):
        got_pages = ops.KVPages(c.k.clone(), c.v.clone(), c.pages.tables, c.page_size, c.ring_pages)
        got = ops.attention(c.qkv, b, got_pages, new_kv=c.new_kv(), kind="decode", keys_per_split=ks, rotate_and_write=rw,
                            **c.kw(softcap=9.0))
        assert_close(got, want, torch.bfloat16, rel=6.0, what=f"output, keys_per_split={ks}")
        assert torch.equal(c.qkv, rows_before), "the packed rows must stay as the projection left them"
        # value rows are copied (equal bits); key rows are rotated in float and rounded once, as the reference does
        assert torch.equal(got_pages.v, ref_pages.v)
        assert_close(got_pages.k, ref_pages.k, torch.bfloat16, rel=1.0, what="key cache")


@pytest.mark.parametrize("sizes", [dict(past=1000, window=400, n_heads=2, n_kv_heads=1, head_dim=64),
                                   dict(past=6000, window=4096, n_heads=8, n_kv_heads=4, head_dim=256),
                                   dict(past=4500, window=4096, n_heads=32, n_kv_heads=16, head_dim=128)])
def test_attention_finds_one_far_key(sizes):
    """One key among thousands is made to dominate: the output must be that key's value row.
    Shows a wrong page, a missed split or a window edge that random data would average away.  The larger
    cases have the real window of 4,096 on a ring of 65 pages that has wrapped."""
    past, W = sizes["past"], sizes["window"]
    nh, nkv, hd = sizes["n_heads"], sizes["n_kv_heads"], sizes["head_dim"]
    G = nh // nkv
    for window, far in ((None, 3), (W, past + 1 - W), (W, past - W), (W, past - 1), (W, past + 1 - W + 64)):
        c = Case(past=[past], new=[1], n_heads=nh, n_kv_heads=nkv, head_dim=hd, page_size=64, window=window,
                 dtype=torch.bfloat16, seed=50, max_context=8192)
        b = c.batch("all")
        page, r = ref._cache_index(c.pages.tables[0], far, c.page_size, c.ring_pages)
        g = nkv - 1                                 # the last kv head: its query heads are the last G
        c.qkv[0, (nh - G) * hd:nh * hd] = 0.25 * (64 / hd) ** 0.5
        c.k[page, g, r] = 8.0 * (64 / hd) ** 0.5    # score 128 against about 0 +- 4 elsewhere
        # the loops of the reference take minutes over thousands of keys and dozens of heads: there the plain
        # kernel (itself compared with the reference above and in the small case here) stands in
        want = (ref.attention(c.qkv, b, c.pages, **c.kw(scale=1.0)) if past <= 2000 else
                ops.attention(c.qkv, b, c.pages, kind="plain", **c.kw(scale=1.0)))
        visible = window is None or past - far < window
        target = ref.cache_load(c.v[page, g, r], r).double().cpu()
        hit = (want[0, (nh - 1) * hd:].double().cpu() - target).abs().max().item() < 1e-2
        assert hit == visible, (window, far)
        for kind in ("decode", "plain"):
            got = ops.attention(c.qkv, b, c.pages, kind=kind, **c.kw(scale=1.0))
            assert_close(got, want, torch.bfloat16, rel=6.0, what=f"{kind} window={window} key={far}")


@pytest.mark.parametrize("kind", ["prefill", "prefill_tc", "plain"])
@pytest.mark.parametrize("window", [None, 200])
def test_prefill_attention_finds_one_key(kind, window):
    """The many-token kernels with one key made to dominate one query's scores: at the window's inner and
    outer edge, and in the first and the last key tile that a query tile of 128 rows reads.  A kernel
    that is off by one at the window's edge, skips a key tile too many or reads a tile twice gives another
    row than the reference; random data would average that away."""
    n = 700
    hd, nh = 64, 2
    for query in (127, 128, 390, 511, 699):
        if window is None:
            keys = [0, 63, 64, query - 1, query]
        else:
            lo = max(query - window + 1, 0)
            keys = sorted({max(lo - 1, 0), lo, lo + 1, min((lo // 64 + 1) * 64, query), query - 1, query})
        for key in keys:
            c = Case(past=[0], new=[n], n_heads=nh, n_kv_heads=1, head_dim=hd, page_size=64, window=window,
                     dtype=torch.bfloat16, seed=52)
            q_cols, k_col = nh * hd, nh * hd
            c.qkv[query, :q_cols] = 0.25
            c.qkv[key, k_col:k_col + hd] = 8.0          # score 128 against about 0 +- 4 elsewhere
            b = c.batch("past")
            # The plain kernel gives the expected rows (the reference's loops over 700 rows take a minute); that it
            # is right itself at this query and key is what `hit == visible` checks, for every kind.
            want = ops.attention(c.qkv, b, c.pages, new_kv=c.new_kv(), kind="plain", **c.kw(scale=1.0))
            visible = key <= query and (window is None or query - key < window)
            target = c.qkv[key, k_col + hd:k_col + 2 * hd].double().cpu()
            got = ops.attention(c.qkv, b, c.pages, new_kv=c.new_kv(), kind=kind, **c.kw(scale=1.0))
            hit = (got[query, :hd].double().cpu() - target).abs().max().item() < 1e-2
            assert hit == visible, (kind, query, key, window)
            assert_close(got, want, torch.bfloat16, rel=6.0, what=f"{kind} window={window} query={query} key={key}")


def test_prefill_attention_on_a_cached_prefix_finds_one_key():
    """The same with the key in the cache (a portion of a prompt on top of earlier steps): the key is put on the
    far side and on the near side of the window's edge, on a ring of pages that has wrapped."""
    window = 100
    for past, key in ((500, 500 + 20 - 99), (500, 500 + 20 - 100), (500, 470), (130, 60)):
        c = Case(past=[past], new=[70], n_heads=2, n_kv_heads=1, head_dim=64, page_size=16, window=window,
                 dtype=torch.bfloat16, seed=53)
        query = 20                                       # row of the portion; its position is past + 20
        page, r = ref._cache_index(c.pages.tables[0], key, c.page_size, c.ring_pages)
        c.qkv[query, :128] = 0.25
        c.k[page, 0, r] = 8.0
        b = c.batch("past")
        want = ref.attention(c.qkv, b, c.pages, new_kv=c.new_kv(), **c.kw(scale=1.0))
        visible = past + query - key < window
        target = ref.cache_load(c.v[page, 0, r], r).double().cpu()
        hit = (want[query, :64].double().cpu() - target).abs().max().item() < 1e-2
        assert hit == visible, (past, key)
        for kind in ("prefill", "plain"):
            got = ops.attention(c.qkv, b, c.pages, new_kv=c.new_kv(), kind=kind, **c.kw(scale=1.0))
            assert_close(got, want, torch.bfloat16, rel=6.0, what=f"{kind} past={past} key={key}")


# ------------------------------------------------------------------------------------------
# sampling
# ------------------------------------------------------------------------------------------

def test_uniform_matches_host():
    from rust_deeplearning_b200.kernels import library
    lib = library.load()
    for seed, stream, step in [(0, 0, 0), (1, 2, 3), (2**63 + 5, 77, 1000), (123456789, 2**40, 2**31)]:
        assert lib.rdl_sampling_uniform(seed, stream, step) == np.float32(uniform_for(seed, stream, step))


@pytest.mark.parametrize("vocab", [131, 40000, 100003, 256000, 300001])
def test_sampling(vocab):
    """Vocabularies of one, two, four and eight blocks a row (32,768 elements each) of the on-chip sampler, and one
    too long for it (the one-block-a-row kernel)."""
    rows = 5
    logits = rnd((rows, vocab), torch.float32, 60, 3.0)
    logits[1, 7] = logits[1, 100] = logits[1].max() + 1.0          # a tie: the first maximum wins
    got = ops.sample(logits, temperature=0.0)
    assert got.tolist() == ref.sample(logits, temperature=0.0).tolist()
    assert got[1].item() == 7
    # equal maxima far apart (in different blocks where a cluster shares the row): the smaller index wins; a maximum at the row's end
    logits[2, vocab - 3] = logits[2, 40] = logits[2].max() + 1.0
    logits[3, vocab - 1] = logits[3].max() + 1.0
    got = ops.sample(logits, temperature=0.0)
    assert got[2].item() == 40 and got[3].item() == vocab - 1
    assert got.tolist() == ref.sample(logits, temperature=0.0).tolist()
    stream = torch.arange(rows, dtype=torch.int64, device=DEV) + 10
    for step in range(3):
        steps = torch.full((rows,), step, dtype=torch.int32, device=DEV)
        hist = torch.randint(0, vocab, (rows * 6,), dtype=torch.int32, device=DEV)
        starts = torch.arange(0, rows * 6 + 1, 6, dtype=torch.int32, device=DEV)
        for kw in (dict(), dict(top_k=7), dict(top_p=0.6), dict(top_k=50, top_p=0.9, repetition_penalty=1.3)):
            args = dict(temperature=0.8, seed=99, row_stream=stream, row_step=steps, history=hist, history_start=starts, **kw)
            got = ops.sample(logits, **args).tolist()
            want = ref.sample(logits, **args).tolist()
            assert got == want, (kw, step, got, want)


@pytest.mark.parametrize("vocab", [256, 40000])
def test_sampling_takes_minus_zero_for_zero(vocab):
    """Logits that are +0 and -0 in turn are all equal: the thresholds of top-k and top-p (found on bit patterns)
    keep all of them, as a comparison of values does."""
    rows = 4
    logits = torch.zeros((rows, vocab), dtype=torch.float32, device=DEV)
    logits[:, ::2] = -0.0
    logits[1, 5] = 1.0
    stream = torch.arange(rows, dtype=torch.int64, device=DEV)
    steps = torch.zeros(rows, dtype=torch.int32, device=DEV)
    hist = torch.zeros(0, dtype=torch.int32, device=DEV)
    starts = torch.zeros(rows + 1, dtype=torch.int32, device=DEV)
    for kw in (dict(top_k=7), dict(top_p=0.5), dict(top_k=3, top_p=0.9)):
        for seed in (1, 2, 3):
            args = dict(temperature=0.7, seed=seed, row_stream=stream, row_step=steps, history=hist, history_start=starts, **kw)
            assert ops.sample(logits, **args).tolist() == ref.sample(logits, **args).tolist(), (kw, seed)


def test_sampling_writes_pinned_host_memory_and_upload_takes_fed_tokens():
    """The sampler's tokens arrive in pinned host memory without a copy of its own; the kernel that brings a step's
    batch description to the device puts the tokens of an earlier sampling in place on the way."""
    logits = rnd((6, 140000), torch.float32, 61, 3.0)
    for kw in (dict(temperature=0.0), dict(temperature=0.8, top_k=20, seed=5)):
        host = torch.full((8,), -1, dtype=torch.int32).pin_memory()
        got = ops.sample(logits, host_out=host, **kw)
        torch.cuda.synchronize()
        assert host[:6].tolist() == got.tolist() and host[6:].tolist() == [-1, -1]
    n = 4096 + 64
    src = torch.arange(n, dtype=torch.int32).pin_memory()
    sampled = torch.tensor([100, 200, 300, 400, 500], dtype=torch.int32, device=DEV)
    tokens_at, token_src_at, n_fed = 8, 2000, 3
    src[token_src_at:token_src_at + n_fed] = torch.tensor([4, 0, 2], dtype=torch.int32)
    dst = torch.full((n,), -7, dtype=torch.int32, device=DEV)
    ops.upload_batch(dst, src, n)
    assert torch.equal(dst.cpu(), src)
    dst.fill_(-7)
    ops.upload_batch(dst, src, n - 64, (sampled, token_src_at, tokens_at, n_fed))
    want = src.clone()
    want[tokens_at:tokens_at + n_fed] = torch.tensor([500, 100, 300], dtype=torch.int32)
    want[n - 64:] = -7
    assert torch.equal(dst.cpu(), want)
