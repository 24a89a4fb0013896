"""Whole-model logits at real layer sizes: two-layer models (one windowed layer, one global) with the
widths of the 2B shape (hidden 2304, 8 heads on 4, head size 256, intermediate 9216), of the 9B shape
(hidden 3584, 16 heads on 8, head size 256, intermediate 14336) and of the 27B shape (hidden 4608, 32
heads on 16, head size 128, query scale 144; intermediate 12288, a third of the real one), the
vocabulary cut to a few thousand so that the plain implementation stays affordable.  At these sizes the engine takes the kernels the tiny
configurations never reach: the tensor-memory prefill attention, the decode kernel's fixed-size forms,
both forms of the tcgen05 product (single blocks and pairs, sums of more than 4,096 terms).

The 32-bit engine is compared with the plain implementation; the bfloat16 engine with both, in the four
cuts, on a request longer than the window plus two pages, so that the window's ring of 64-row pages wraps
in a whole prompt, in a portion on a cached prefix and in single-token steps.  A second case has the real
window of 4,096 with a request of 4,200 tokens and 40 single-token steps; there the 32-bit engine is the
reference (the plain implementation would take minutes).
"""
import functools
import os

import numpy as np
import pytest
import torch

import model_helpers as mh
import plain_gemma2 as plain

pytestmark = pytest.mark.gpu
REAL_BF16 = 0.005      # bfloat16 tolerance as a fraction of the largest logit: observed 0.0015 to 0.0019 at the three widths

WIDTHS = {
    "2b": dict(hidden_size=2304, num_attention_heads=8, num_key_value_heads=4, head_dim=256, intermediate_size=9216,
               query_pre_attn_scalar=256, vocab_size=4096),
    "9b": dict(hidden_size=3584, num_attention_heads=16, num_key_value_heads=8, head_dim=256, intermediate_size=14336,
               query_pre_attn_scalar=256, vocab_size=3500),
    "27b": dict(hidden_size=4608, num_attention_heads=32, num_key_value_heads=16, head_dim=128, intermediate_size=12288,
                query_pre_attn_scalar=144, vocab_size=3000),
}


def config(shape, window):
    cfg = {"architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2", "num_hidden_layers": 2,
           "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "sliding_window": window,
           "attn_logit_softcapping": 50.0, "final_logit_softcapping": 30.0, "max_position_embeddings": 8192,
           "hidden_activation": "gelu_pytorch_tanh", "tie_word_embeddings": True, "bos_token_id": 2, "eos_token_id": 1}
    cfg.update(WIDTHS[shape])
    return cfg


@functools.lru_cache(maxsize=None)
def folder(shape):
    """The model with a window of 1,024 as a folder (weights made on the device, the same numbers the host makes)."""
    from rust_deeplearning_b200 import write_random_model
    path = os.path.join(mh.tmp_root(), f"real_{shape}")
    write_random_model(path, config(shape, 1024), 11, "bfloat16", device="cuda:0")
    return path


@functools.lru_cache(maxsize=2)
def loaded(shape, dtype):
    from rust_deeplearning_b200 import load_model
    return load_model(folder(shape), dtype)


@functools.lru_cache(maxsize=None)
def sequences(shape):
    V = WIDTHS[shape]["vocab_size"]
    return [mh.prompt(950, 1300, V), mh.prompt(951, 200, V), mh.prompt(952, 70, V)]


@functools.lru_cache(maxsize=None)
def _all_plain_logits(shape):
    cfg, w = plain.load_folder(folder(shape))          # float64 copies of the weights: dropped again after this call
    return [plain.forward(cfg, w, ids) for ids in sequences(shape)]


def plain_logits(shape, which):
    return _all_plain_logits(shape)[which]


def report(what, got, want):
    err = (got.detach().double().cpu().numpy() - want).__abs__().max()
    print(f"[real sizes] {what}: largest logit {np.abs(want).max():.3f}, largest error {err:.3e}")
    return err


@pytest.mark.parametrize("shape", ["2b", "9b", "27b"])
def test_float32_engine_against_the_plain_implementation(shape):
    from rust_deeplearning_b200 import Engine
    eng = Engine(loaded(shape, "float32"), max_tokens=2048)
    ids = sequences(shape)[0]
    want = plain_logits(shape, 0)
    slot = eng.new_sequence()
    whole = eng.step([slot], [ids], "all").clone()
    report(f"{shape} float32 whole", whole, want)
    mh.assert_logits(whole, want, "float32", f"{shape} float32, 1300 tokens whole")
    eng.release(slot)
    # the last 32 one by one: the ring (window 1024, 18 pages of 64) wraps; bit-equal to the whole run
    slot = eng.new_sequence()
    first = eng.step([slot], [ids[:1268]], "all").clone()
    assert torch.equal(first, whole[:1268])
    for t in range(1268, 1300):
        assert torch.equal(eng.step([slot], [[ids[t]]], "all"), whole[t:t + 1]), f"position {t} differs from the whole run"


@pytest.mark.parametrize("shape", ["2b", "9b", "27b"])
def test_bfloat16_engine_in_four_cuts(shape):
    from rust_deeplearning_b200 import Engine
    eng = Engine(loaded(shape, "bfloat16"), max_tokens=4096, max_seqs=4)
    seqs = sequences(shape)
    want = [plain_logits(shape, i) for i in range(3)]
    ids = seqs[0]
    # 1. whole: the tensor-memory attention, tcgen05 products
    slot = eng.new_sequence()
    got = eng.step([slot], [ids], "all")
    report(f"{shape} bfloat16 whole", got, want[0])
    mh.assert_logits(got, want[0], "bfloat16", f"{shape} whole", bf16_fraction=REAL_BF16)
    eng.release(slot)
    # 2. the last 32 one by one: weight-streaming products, decode attention on a wrapped ring
    slot = eng.new_sequence()
    eng.step([slot], [ids[:1268]], [[]])
    rows = [eng.step([slot], [[ids[t]]], "last").clone() for t in range(1268, 1300)]
    report(f"{shape} bfloat16 last 32 one by one", torch.cat(rows), want[0][1268:])
    mh.assert_logits(torch.cat(rows), want[0][1268:], "bfloat16", f"{shape} last 32 one by one", bf16_fraction=REAL_BF16)
    eng.release(slot)
    # 3. in portions: 700 + 500 + 100 tokens; the second and third read a cached prefix on the wrapped ring
    slot = eng.new_sequence()
    parts = [eng.step([slot], [ids[a:b]], "all").clone() for a, b in ((0, 700), (700, 1200), (1200, 1300))]
    report(f"{shape} bfloat16 portions", torch.cat(parts), want[0])
    mh.assert_logits(torch.cat(parts), want[0], "bfloat16", f"{shape} portions", bf16_fraction=REAL_BF16)
    eng.release(slot)
    # 4. a batch of unequal lengths, the shorter requests ending earlier, then the next batch on their slots
    for round_ in range(2):
        cut = [len(s) - k for s, k in zip(seqs, (6, 3, 9))]
        slots = [eng.new_sequence() for _ in seqs]
        got = eng.step(slots, [s[:c] for s, c in zip(seqs, cut)], "last")
        mh.assert_logits(got, np.stack([w[c - 1] for w, c in zip(want, cut)]), "bfloat16", f"{shape} batch prompts", bf16_fraction=REAL_BF16)
        pos = list(cut)
        live = [0, 1, 2]
        while live:
            got = eng.step([slots[i] for i in live], [[seqs[i][pos[i]]] for i in live], "last")
            mh.assert_logits(got, np.stack([want[i][pos[i]] for i in live]), "bfloat16", f"{shape} batch decode at {pos}", bf16_fraction=REAL_BF16)
            for i in live:
                pos[i] += 1
            for i in [i for i in live if pos[i] == len(seqs[i])]:
                eng.release(slots[i])
            live = [i for i in live if pos[i] < len(seqs[i])]
    assert eng.graph_replays > 0


@pytest.mark.parametrize("shape", ["2b", "27b"])
def test_window_of_4096_wraps_its_ring(shape):
    """The real window: 4,200 tokens (66 ring entries of 64 rows wrap) whole and in two portions, then 40
    single tokens; bfloat16 against the 32-bit engine on the same weights."""
    from rust_deeplearning_b200 import Engine, random_model
    cfg = config(shape, 4096)
    ids = mh.prompt(960, 4240, cfg["vocab_size"])
    ref = Engine(random_model(cfg, 12, "float32"), max_tokens=4352, max_seqs=1)
    assert any(g.is_ring and g.ring_pages * 64 < 4240 for g in ref.cache.kv_groups)      # the ring wraps
    slot = ref.new_sequence()
    want = [ref.step([slot], [ids[:4200]], [[0, 100, 4095, 4096, 4097, 4199]]).double().cpu().numpy()]
    want += [ref.step([slot], [[ids[t]]], "last").double().cpu().numpy() for t in range(4200, 4240)]
    want = np.concatenate(want)
    del ref
    torch.cuda.empty_cache()
    eng = Engine(random_model(cfg, 12, "bfloat16"), max_tokens=2 * 4352, max_seqs=2)
    for portions in ([(0, 4200)], [(0, 2100), (2100, 4200)]):
        slot = eng.new_sequence()
        got = []
        for a, b in portions:
            places = [p - a for p in (0, 100, 4095, 4096, 4097, 4199) if a <= p < b]
            got.append(eng.step([slot], [ids[a:b]], [places]).clone())
        got += [eng.step([slot], [[ids[t]]], "last").clone() for t in range(4200, 4240)]
        report(f"{shape} window 4096, portions {portions}", torch.cat(got), want)
        mh.assert_logits(torch.cat(got), want, "bfloat16", f"{shape} window 4096 {portions}", bf16_fraction=REAL_BF16)
        eng.release(slot)


@pytest.mark.parametrize("case", range(9))
def test_batches_drawn_at_random_against_the_32_bit_engine(case):
    """1 to 24 sequences (the split norms' 8-row and 16-row operands, the weight-streaming product without them, the
    library product from 17 rows) of 2 to 1,500 tokens at the three widths, prompts whole or in portions of up to
    600 tokens that mix with one another, then the last 1 to 7 tokens one by one with the shorter sequences ending
    earlier: the bfloat16 engine's logits against the 32-bit engine's."""
    from rust_deeplearning_b200 import Engine
    rng = np.random.default_rng(case)
    shape = ["2b", "27b", "9b"][case % 3]
    V = WIDTHS[shape]["vocab_size"]
    n = int(rng.choice([1, 3, 4, 5, 8, 9, 16, 17, 24]))
    lengths = [int(v) for v in rng.integers(2, 1500 if n <= 8 else 400, size=n)]
    k = int(rng.integers(1, 8))
    cut = [max(1, n_tokens - k) for n_tokens in lengths]
    portions = bool(rng.integers(0, 2))
    seqs = [mh.prompt(9000 + 50 * case + i, n_tokens, V) for i, n_tokens in enumerate(lengths)]
    outs = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine(loaded(shape, dtype), max_tokens=24 * 1536, max_seqs=24)
        slots = [eng.new_sequence() for _ in seqs]
        rows = []
        if portions:
            pos, draw = [0] * n, np.random.default_rng(case + 1)
            while any(p < c for p, c in zip(pos, cut)):
                live = [i for i in range(n) if pos[i] < cut[i]]
                toks = [seqs[i][pos[i]:min(cut[i], pos[i] + int(draw.integers(1, 600)))] for i in live]
                rows.append(eng.step([slots[i] for i in live], toks, "last").clone())
                for i, t in zip(live, toks):
                    pos[i] += len(t)
        else:
            rows.append(eng.step(slots, [s[:c] for s, c in zip(seqs, cut)], "last").clone())
        pos = list(cut)
        while True:
            live = [i for i in range(n) if pos[i] < lengths[i]]
            if not live:
                break
            rows.append(eng.step([slots[i] for i in live], [[seqs[i][pos[i]]] for i in live], "last").clone())
            for i in live:
                pos[i] += 1
        eng.check_status()
        outs[dtype] = torch.cat(rows)
        del eng
    want = outs["float32"].double().cpu().numpy()
    report(f"{shape}, {n} sequences, bfloat16 against float32", outs["bfloat16"], want)
    mh.assert_logits(outs["bfloat16"], want, "bfloat16", f"{shape}, {n} sequences of {lengths[:6]}, portions {portions}", bf16_fraction=REAL_BF16)
