"""The attention kernels on geometry drawn at random (seeded): one to five sequences, cached prefixes of up to
1,500 keys and up to 700 new rows, head sizes from 16 to 256, one to four key/value heads with one to eight query
heads each, windows from 5 keys to none, pages of 8 to 64 rows, page lists in random order, soft-cap on and off, two
score scales - for the decode kernel (also rotating and writing the new rows itself), the prefill kernel on a cached
prefix and the tcgen05 prefill kernel.  The reference is `kernel_refs.attention_vectorised`, which the first test
holds against the key-by-key reference on small cases."""
import math

import numpy as np
import pytest
import torch

import kernel_refs as ref
from rust_deeplearning_b200.kernels import ops
from test_kernels_gpu import Case, assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
KINDS = ["decode", "prefill", "prefill_tc", "decode_rotating"]


def draw(case: int, small: bool = False):
    rng = np.random.default_rng(case)
    kind = KINDS[case % 4]
    n = int(rng.integers(1, 6))
    n_kv = int(rng.choice([1, 2, 3, 4]))
    group = int(rng.choice([1, 2, 3, 4, 5, 8]))
    window = int(rng.choice([0, 0, 5, 33, 64, 100, 129, 500, 1024, 2000]))
    softcap = float(rng.choice([0, 5.0, 30.0])) or None
    most = 40 if small else None
    if kind.startswith("decode"):
        hd, page = int(rng.choice([16, 32, 48, 64, 80, 128, 192, 256])), int(rng.choice([16, 32, 48, 64]))
        past, new = [int(v) for v in rng.integers(0, most or 1500, size=n)], [1] * n
    elif kind == "prefill":
        hd, page = int(rng.choice([16, 32, 48, 64, 80, 128, 256])), int(rng.choice([8, 16, 32, 64]))
        past = [int(v) * int(rng.integers(0, 2)) for v in rng.integers(0, most or 600, size=n)]
        new = [int(v) for v in rng.integers(1, most or 300, size=n)]
    else:
        hd, page = int(rng.choice([64, 128, 192, 256])), 64
        past, new = [0] * n, [int(v) for v in rng.integers(1, most or 700, size=n)]
    c = Case(past=past, new=new, n_heads=n_kv * group, n_kv_heads=n_kv, head_dim=hd, page_size=page, window=window or None,
             dtype=torch.bfloat16, seed=100 + case)
    kw = c.kw(scale=float(rng.choice([1.0, 3.0])) / math.sqrt(hd), softcap=softcap)
    what = f"{kind}: heads {n_kv * group}/{n_kv} x {hd}, page {page}, window {window}, soft-cap {softcap}, cached {past}, new {new}"
    return rng, kind, c, kw, what


@pytest.mark.parametrize("case", range(12))
def test_the_vectorised_reference_is_the_key_by_key_one(case):
    _, kind, c, kw, what = draw(case, small=True)
    if kind.startswith("decode"):
        b, new_kv = c.batch("all"), None
    else:
        b, new_kv = c.batch("past"), c.new_kv()
    assert_close(ref.attention_vectorised(c.qkv, b, c.pages, new_kv=new_kv, **kw), ref.attention(c.qkv, b, c.pages, new_kv=new_kv, **kw),
                 torch.bfloat16, rel=1.0, what=what)


@pytest.mark.parametrize("first", range(0, 160, 16))
def test_attention_on_geometry_drawn_at_random(first):
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for case in range(first, first + 16):
        rng, kind, c, kw, what = draw(case)
        if kind == "decode":
            b = c.batch("all")
            ks = [None, c.page_size, 8 * c.page_size][int(rng.integers(0, 3))]
            got = ops.attention(c.qkv, b, c.pages, kind="decode", keys_per_split=ks, status=status, **kw)
            want = ref.attention_vectorised(c.qkv, b, c.pages, **kw)
        elif kind == "decode_rotating":
            b, hd = c.batch("all"), c.head_dim
            rot = [hd, hd // 2, 0][int(rng.integers(0, 3))]
            rot = rot if rot % 16 == 0 else 0
            half = max(rot // 2, 1)
            ang = torch.arange(int(c.seq_end.max()) + 1, dtype=torch.float64)[:, None] / (50.0 ** (torch.arange(half, dtype=torch.float64) / half))
            cos, sin = ang.cos().float().to(DEV).contiguous(), ang.sin().float().to(DEV).contiguous()
            want_pages = ops.KVPages(c.k.clone(), c.v.clone(), c.pages.tables, c.page_size, c.ring_pages)
            rotated = c.qkv.clone()
            ref.rope_cache(rotated, c.n_heads, c.n_kv_heads, hd, tok_seq=b.tok_seq, tok_pos=b.tok_pos, cos=cos if rot else None,
                           sin=sin if rot else None, rotary_dim=rot, pages=want_pages, seq_end=b.seq_cached)
            want = ref.attention_vectorised(rotated, b, want_pages, **kw)
            got_pages = ops.KVPages(c.k.clone(), c.v.clone(), c.pages.tables, c.page_size, c.ring_pages)
            got = ops.attention(c.qkv, b, got_pages, new_kv=c.new_kv(), kind="decode", status=status,
                                rotate_and_write=(cos, sin, rot) if rot else (None, None, 0), **kw)
            assert torch.equal(got_pages.v, want_pages.v), f"value cache; {what}"
            assert_close(got_pages.k, want_pages.k, torch.bfloat16, rel=1.0, what=f"key cache; {what}")
        else:
            b = c.batch("past")
            got = ops.attention(c.qkv, b, c.pages, new_kv=c.new_kv(), kind=kind, status=status, **kw)
            want = ref.attention_vectorised(c.qkv, b, c.pages, new_kv=c.new_kv(), **kw)
        assert_close(got, want, torch.bfloat16, rel=6.0, what=what)
        assert status.item() == 0, what
