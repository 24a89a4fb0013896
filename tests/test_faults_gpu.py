"""What the library does when a kernel cannot finish its work, tested without faulting or hanging anything:
every kernel of a step receives the engine's status word; a token id outside the vocabulary that arrives
from the device is reported; a bounded wait that is made to run out (a short limit, and a barrier told to
expect more bytes than its copy delivers) ends with the kernel's own code in the status word, a normal
return, clean run counters and a correct next launch."""
import ctypes

import numpy as np
import pytest
import torch

import kernel_refs as ref
import model_helpers as mh
import tiny_configs
from rust_deeplearning_b200.kernels import library, ops
from test_kernels_gpu import Case, assert_close, rnd

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SHORT_WAIT = 200_000       # clock cycles, about a tenth of a millisecond: every copy has long arrived


def _value(arg):
    return arg.value if isinstance(arg, ctypes.c_void_p) else arg


def test_every_kernel_of_a_step_gets_the_status_word(monkeypatch):
    """Embedding, both kinds of matrix product and the attention kernels that can report a fault are called
    with the address of the engine's status word, in prompt steps and in single-token steps."""
    lib = library.load()
    seen = {}

    def watch(name, status_of):
        orig = getattr(lib, name)

        def wrapper(*args):
            seen.setdefault(name, []).append(status_of(args))
            return orig(*args)
        monkeypatch.setattr(lib, name, wrapper)

    watch("rdl_embed_rows", lambda a: _value(a[8]))
    watch("rdl_gemm_skinny", lambda a: _value(a[10]))
    watch("rdl_gemm_tc", lambda a: _value(a[10]))
    watch("rdl_gemm_skinny_norm", lambda a: _value(a[11]))      # the products that carry the norms in single-token steps
    watch("rdl_attention_decode", lambda a: a[0]._obj.status)
    watch("rdl_attention_prefill_tc", lambda a: a[0]._obj.status)
    name = "D"                                     # head size 64: the tcgen05 prefill attention takes its prompts
    eng = mh.engine(name, "bfloat16", use_graphs=False)
    V = tiny_configs.config(name)[0]["vocab_size"]
    ids = mh.prompt(800, 150, V)
    slot = eng.new_sequence()
    eng.step([slot], [ids[:140]], "last")           # 140 rows: tcgen05 products and attention
    eng.step([slot], [ids[140:149]], "last")        # 9 rows: the weight-streaming product
    eng.step([slot], [[ids[149]]], "last")          # one row: the decode attention
    torch.cuda.synchronize()
    word = eng.status.data_ptr()
    for kernel in ("rdl_embed_rows", "rdl_gemm_skinny", "rdl_gemm_skinny_norm", "rdl_gemm_tc", "rdl_attention_decode",
                   "rdl_attention_prefill_tc"):
        assert kernel in seen, f"{kernel} was not launched"
        assert all(s == word for s in seen[kernel]), f"{kernel} was launched without the engine's status word"
    eng.check_status()


def test_a_bad_token_id_from_the_device_is_reported_and_the_engine_goes_on():
    name = "A"
    eng = mh.engine(name, "float32", use_graphs=False)
    V = tiny_configs.config(name)[0]["vocab_size"]
    ids = mh.prompt(801, 9, V)
    want = mh.plain_logits(name, ids)
    slot = eng.new_sequence()
    eng.step([slot], [ids[:8]], "last")
    sampled = torch.tensor([V + 5], dtype=torch.int32, device=DEV)       # what a broken sampler might hand over
    logits = eng.step([slot], None, "last", fed=(sampled, [0]))
    assert torch.isnan(logits).all()                                      # never a wrong result: the row is poisoned
    with pytest.raises(RuntimeError, match="embed_rows"):
        eng.check_status()
    eng.check_status()                                                    # the word was cleared
    eng.release(slot)
    slot = eng.new_sequence()
    mh.assert_logits(eng.step([slot], [ids], "all"), want, "float32", "after the fault")


def test_decode_attention_wait_runs_out():
    lib = library.load()
    c = Case(past=[700, 130], new=[1, 1], n_heads=8, n_kv_heads=4, head_dim=128, page_size=64, window=None,
             dtype=torch.bfloat16, seed=81)
    b = c.batch("all")
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    need = lib.rdl_attention_decode_scratch_bytes(c.T, c.n_heads, c.n_kv_heads, c.head_dim, 16)
    scratch = torch.zeros(need // 4 + 64, dtype=torch.float32, device=DEV)
    counters = lib.rdl_attention_decode_counter_bytes(c.T, c.n_kv_heads) // 4
    want = ref.attention(c.qkv, b, c.pages, **c.kw(softcap=7.0))
    try:
        lib.rdl_set_wait_test(3, SHORT_WAIT, 64)
        ops.attention(c.qkv, b, c.pages, kind="decode", keys_per_split=c.page_size, scratch=lambda n: scratch,
                      status=status, **c.kw(softcap=7.0))
        torch.cuda.synchronize()                   # the kernel returned by itself
    finally:
        lib.rdl_set_wait_test(0, 0, 0)
    assert status.item() == 3
    assert not scratch[:counters].view(torch.int32).any(), "the run counters must be left at zero"
    status.zero_()
    got = ops.attention(c.qkv, b, c.pages, kind="decode", keys_per_split=c.page_size, scratch=lambda n: scratch,
                        status=status, **c.kw(softcap=7.0))
    assert_close(got, want, torch.bfloat16, rel=6.0, what="the launch after the fault")
    assert status.item() == 0


def test_weight_streaming_product_wait_runs_out():
    lib = library.load()
    x, w = rnd((8, 512), torch.bfloat16, 82), rnd((300, 512), torch.bfloat16, 83, 0.2)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    try:
        lib.rdl_set_wait_test(7, SHORT_WAIT, 64)
        ops.linear(x, w, status=status)
        torch.cuda.synchronize()
    finally:
        lib.rdl_set_wait_test(0, 0, 0)
    assert status.item() == 7
    status.zero_()
    assert_close(ops.linear(x, w, status=status), ref.linear(x, w), torch.bfloat16, what="the launch after the fault")
    assert status.item() == 0


def test_engine_names_the_kernel_that_gave_up():
    """Through the engine: a single-token step whose decode attention gives up raises from check_status with
    the kernel's name; the sequence is dropped, and the next sequence's steps (on the same scratch) are right."""
    lib = library.load()
    name = "B"
    eng = mh.engine(name, "bfloat16", use_graphs=False)
    V = tiny_configs.config(name)[0]["vocab_size"]
    ids = mh.prompt(802, 40, V)
    want = mh.plain_logits(name, ids)
    slot = eng.new_sequence()
    eng.step([slot], [ids[:30]], "last")
    try:
        lib.rdl_set_wait_test(3, SHORT_WAIT, 64)
        logits = eng.step([slot], [[ids[30]]], "last")
        logits.cpu()
    finally:
        lib.rdl_set_wait_test(0, 0, 0)
    with pytest.raises(RuntimeError, match="attention_decode"):
        eng.check_status()
    eng.release(slot)                                # its cache rows of that step are void
    slot = eng.new_sequence()
    mh.assert_logits(eng.step([slot], [ids[:30]], "all"), want[:30], "bfloat16", "prompt after the fault")
    for t in range(30, 40):
        mh.assert_logits(eng.step([slot], [[ids[t]]], "last"), want[t:t + 1], "bfloat16", f"position {t} after the fault")
    eng.check_status()
