"""The entry point for callers that cannot allocate, `rdl_attention_decode_static`, called through
its exported C symbol: decode attention whose scratch is a fixed array inside the library.  A host
that has given all device memory to the cache, or that may not call cudaMalloc inside its serving
loop, uses it in place of `rdl_attention_decode`.  It must give what the ordinary entry point
gives, call after call on the shared array, and refuse what does not fit.

This file sorts last on purpose: a run that stops at the first failure has then run every other test."""
import ctypes

import pytest
import torch

import kernel_refs as ref
from rust_deeplearning_b200.kernels import library, ops
from test_kernels_gpu import Case, assert_close

pytestmark = pytest.mark.gpu


def static_decode(case, batch, keys_per_split, softcap):
    """Fill the argument structure as ops.attention does, but pass no scratch."""
    lib = library.load()
    fn = lib.rdl_attention_decode_static
    fn.argtypes = [ctypes.POINTER(library.AttentionArgs), ctypes.c_void_p]
    fn.restype = ctypes.c_int
    q = case.qkv
    out = torch.full((q.shape[0], case.n_heads * case.head_dim), float("nan"), dtype=q.dtype, device=q.device)
    kw = case.kw(softcap=softcap)
    a = ops._attention_args(q.data_ptr(), q.stride(0), None, None, 0, out, batch, case.pages, case.n_heads,
                            case.n_kv_heads, case.head_dim, kw["score_scale"], softcap, case.window)
    a.keys_per_split = keys_per_split
    a.max_splits = (max(batch.max_keys, 1) + keys_per_split - 1) // keys_per_split + 1
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    status = fn(ctypes.byref(a), stream)
    return status, out


SHAPES = [
    dict(past=[0, 63, 64, 700], n_heads=8, n_kv_heads=4, head_dim=256, page_size=64, window=None),
    dict(past=[2000, 17, 130], n_heads=4, n_kv_heads=2, head_dim=128, page_size=64, window=100),
]


def test_static_scratch_entry_point_matches_the_ordinary_one_and_the_plain_reference():
    """Calls in a row on the one shared array, alternating between two shapes (other token counts, head
    counts and numbers of runs), so that what one call leaves in the array - counters, partial sums of
    runs the next call does not have - would show in the next call's result.  Every result is compared
    with the ordinary entry point and with the plain reference of the operation."""
    cases = []
    for k, shape in enumerate(SHAPES):
        shape = dict(shape)
        past = shape.pop("past")
        case = Case(past=past, new=[1] * len(past), dtype=torch.bfloat16, seed=70 + k, **shape)
        cases.append((case, case.batch("all")))
    for call, (which, softcap) in enumerate(((0, None), (1, 7.0), (0, 7.0), (1, None), (1, None))):
        case, batch = cases[which]
        want = ops.attention(case.qkv, batch, case.pages, kind="decode", keys_per_split=case.page_size,
                             **case.kw(softcap=softcap))
        plain = ref.attention(case.qkv, batch, case.pages, **case.kw(softcap=softcap))
        status, got = static_decode(case, batch, case.page_size, softcap)
        assert status == 0, library.load().rdl_last_error().decode()
        torch.cuda.synchronize()
        assert not torch.isnan(got.float()).any(), f"call {call}: rows left unwritten"
        assert_close(got, want, torch.bfloat16, rel=6.0, what=f"call {call} against the ordinary entry point")
        assert_close(got, plain, torch.bfloat16, rel=6.0, what=f"call {call} against the plain reference")


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    past = [3000] * 40
    case = Case(past=past, new=[1] * len(past), n_heads=16, n_kv_heads=2, head_dim=64, page_size=16, window=None,
                dtype=torch.bfloat16, seed=71)
    status, _ = static_decode(case, case.batch("all"), 16, None)     # 40 x 16 heads x 189 runs x 66 floats > 8 MiB
    assert status != 0
    assert b"fixed array" in library.load().rdl_last_error()
