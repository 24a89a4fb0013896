"""Ways of cutting and batching that the other engine tests do not run, on the real kernels, against the
plain implementation: a step that mixes whole prompts with single tokens; prompts fed in portions of many
tokens on top of a cached prefix, on small pages so that the window's ring wraps inside a portion and a
request is left out of a step; and, in 32-bit, logits that are bit-equal however the tokens are cut -
including a step of more than 256 rows, where a kernel that chose its shape by the row count would differ."""
import numpy as np
import pytest
import torch

import model_helpers as mh
import tiny_configs

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def vocab(name):
    return tiny_configs.config(name)[0]["vocab_size"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_a_step_mixes_whole_prompts_and_single_tokens(name, dtype):
    """Two sequences are under way (one of them past the window); a step then brings one token for each of
    them and, in the same batch, two prompts that start at position 0."""
    eng = mh.engine(name, dtype)
    V = vocab(name)
    old = [mh.prompt(700 + i, n, V) for i, n in enumerate((41, 6))]       # under way when the prompts arrive
    new = [mh.prompt(710 + i, n, V) for i, n in enumerate((19, 3))]       # start in the first mixed step
    late = mh.prompt(720, 11, V)                                          # starts in the second
    w_old = [mh.plain_logits(name, s) for s in old]
    w_new = [mh.plain_logits(name, s) for s in new]
    s_old = [eng.new_sequence() for _ in old]
    s_new = [eng.new_sequence() for _ in new]
    eng.step(s_old, [s[:-2] for s in old], [[], []])
    # single token, prompt, single token, prompt
    got = eng.step([s_old[0], s_new[0], s_old[1], s_new[1]], [[old[0][-2]], new[0][:-1], [old[1][-2]], new[1][:-1]], "all")
    want = np.concatenate([w_old[0][-2:-1], w_new[0][:-1], w_old[1][-2:-1], w_new[1][:-1]])
    mh.assert_logits(got, want, dtype, f"{name} first mixed step")
    # four single tokens and one more prompt
    s_late = eng.new_sequence()
    got = eng.step([s_old[0], s_new[0], s_late, s_old[1], s_new[1]],
                   [[old[0][-1]], [new[0][-1]], late, [old[1][-1]], [new[1][-1]]], "all")
    want = np.concatenate([w_old[0][-1:], w_new[0][-1:], mh.plain_logits(name, late), w_old[1][-1:], w_new[1][-1:]])
    mh.assert_logits(got, want, dtype, f"{name} second mixed step")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("page_size,portions", [(16, (7, 2, 60, 1, 80)), (64, (7, 23, 15, 70, 60))])
@pytest.mark.parametrize("name", ["A", "B"])
def test_prompts_in_portions_on_a_cached_prefix(name, dtype, page_size, portions):
    """Two sequences fed in portions of many tokens (the windowed layers' ring wraps inside a portion at 16
    positions a page: 3 pages for a window of 8 or 16 plus slack), the second one left out of the third
    step and fed a portion alone afterwards; then a few single tokens.  Every position against the plain
    implementation."""
    eng = mh.engine(name, dtype, page_size=page_size, max_tokens=1024)
    V = vocab(name)
    total = sum(portions) + 4
    a, b = mh.prompt(730, total, V), mh.prompt(731, total, V)
    wa, wb = mh.plain_logits(name, a), mh.plain_logits(name, b)
    sa, sb = eng.new_sequence(), eng.new_sequence()
    pa = pb = 0
    for k, n in enumerate(portions):
        if k == 2:
            # only the first sequence takes this step; the second catches up alone right after
            mh.assert_logits(eng.step([sa], [a[pa:pa + n]], "all"), wa[pa:pa + n], dtype, f"{name} portion {k} of a alone")
            mh.assert_logits(eng.step([sb], [b[pb:pb + n]], "all"), wb[pb:pb + n], dtype, f"{name} portion {k} of b alone")
        else:
            got = eng.step([sa, sb], [a[pa:pa + n], b[pb:pb + n]], "all")
            mh.assert_logits(got, np.concatenate([wa[pa:pa + n], wb[pb:pb + n]]), dtype, f"{name} portion {k}")
        pa += n
        pb += n
    for t in range(pa, total):
        got = eng.step([sa, sb], [[a[t]], [b[t]]], "last")
        mh.assert_logits(got, np.stack([wa[t], wb[t]]), dtype, f"{name} position {t}")


def _cuts(eng, seqs):
    """The logits of every position of every sequence, computed in four ways; a dict cut -> [per sequence]."""
    out = {}
    # each alone and whole
    res = []
    for s in seqs:
        slot = eng.new_sequence()
        res.append(eng.step([slot], [s], "all").clone())
        eng.release(slot)
    out["whole"] = res
    # each alone, the last 32 one by one
    res = []
    for s in seqs:
        slot = eng.new_sequence()
        cut = max(len(s) - 32, 1)
        parts = [eng.step([slot], [s[:cut]], "all").clone()]
        for t in range(cut, len(s)):
            parts.append(eng.step([slot], [[s[t]]], "all").clone())
        eng.release(slot)
        res.append(torch.cat(parts))
    out["last 32 one by one"] = res
    # all together: prompts (all but the last 5 tokens) in one step, then one token each
    slots = [eng.new_sequence() for _ in seqs]
    cuts = [max(len(s) - 5, 1) for s in seqs]
    first = eng.step(slots, [s[:c] for s, c in zip(seqs, cuts)], "all")
    parts = [[p] for p in torch.split(first.clone(), cuts)]
    pos = list(cuts)
    live = [i for i, s in enumerate(seqs) if pos[i] < len(s)]
    while live:
        got = eng.step([slots[i] for i in live], [[seqs[i][pos[i]]] for i in live], "all").clone()
        for row, i in enumerate(live):
            parts[i].append(got[row:row + 1])
            pos[i] += 1
        live = [i for i in live if pos[i] < len(seqs[i])]
    for sl in slots:
        eng.release(sl)
    out["batch"] = [torch.cat(p) for p in parts]
    # in portions of 23 tokens, two sequences a step where two are left
    slots = [eng.new_sequence() for _ in seqs]
    parts = [[] for _ in seqs]
    pos = [0] * len(seqs)
    live = list(range(len(seqs)))
    while live:
        take = [min(23, len(seqs[i]) - pos[i]) for i in live]
        got = eng.step([slots[i] for i in live], [seqs[i][pos[i]:pos[i] + n] for i, n in zip(live, take)], "all").clone()
        for i, chunk in zip(live, torch.split(got, take)):
            parts[i].append(chunk)
        for i, n in zip(live, take):
            pos[i] += n
        live = [i for i in live if pos[i] < len(seqs[i])]
    for sl in slots:
        eng.release(sl)
    out["portions of 23"] = [torch.cat(p) for p in parts]
    return out


@pytest.mark.parametrize("name", ["A", "B"])
def test_float32_logits_are_bit_equal_across_cuts(name):
    """The 32-bit path sums in an order that depends on positions and sizes of the model alone, so the same
    token at the same position gives the same bits whether it came whole, one by one, in a batch or in
    portions.  One sequence has 300 tokens: its whole-prompt step has more than 256 rows, its single-token
    steps have one."""
    eng = mh.engine(name, "float32", max_tokens=2048)
    V = vocab(name)
    seqs = [mh.prompt(740 + i, n, V) for i, n in enumerate((300, 37, 70))]
    cuts = _cuts(eng, seqs)
    ref = cuts["whole"]
    for i, s in enumerate(seqs):
        mh.assert_logits(ref[i], mh.plain_logits(name, s), "float32", f"{name} sequence {i} whole")
    for cut, res in cuts.items():
        for i in range(len(seqs)):
            same = torch.equal(res[i], ref[i])
            if not same:
                bad = (res[i] != ref[i]).any(dim=1).nonzero()[0].item()
                raise AssertionError(f"{name}, cut '{cut}', sequence {i}: logits differ from the whole run first at "
                                     f"position {bad} (max difference {(res[i] - ref[i]).abs().max().item():.3e})")


@pytest.mark.parametrize("name", ["A", "B"])
def test_bfloat16_cuts_differ_by_rounding_only(name):
    eng = mh.engine(name, "bfloat16", max_tokens=2048)
    V = vocab(name)
    seqs = [mh.prompt(740 + i, n, V) for i, n in enumerate((300, 37, 70))]
    for cut, res in _cuts(eng, seqs).items():
        for i, s in enumerate(seqs):
            mh.assert_logits(res[i], mh.plain_logits(name, s), "bfloat16", f"{name} cut '{cut}' sequence {i}")


@pytest.mark.parametrize("hidden", [2304, 4608, 1000])
def test_float32_norm_rows_do_not_depend_on_the_row_count(hidden):
    """The fused norm at real widths: a float32 row normed in a step of 300 rows, of 8 rows or alone gives
    the same bits (with many rows the bfloat16 path picks another block shape; the 32-bit path must not)."""
    from rust_deeplearning_b200.kernels import ops
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(300, hidden, device="cuda", generator=g)
    res = torch.randn(300, hidden, device="cuda", generator=g)
    w1 = ops.NormParams(torch.randn(hidden, device="cuda", generator=g) * 0.1, 1e-6, 1.0)
    w2 = ops.NormParams(torch.randn(hidden, device="cuda", generator=g) * 0.1, 1e-5, 1.0)
    outs = {}
    for rows in (300, 8, 1):
        r = res[:rows].clone()
        y = ops.norm_residual_norm(x[:rows].contiguous(), first=w1, residual=r, second=w2, out_dtype=torch.float32)
        z = ops.norm_residual_norm(x[:rows].contiguous(), second=w2, out_dtype=torch.float32)
        outs[rows] = (y, r, z)
    for rows in (8, 1):
        for got, want, what in zip(outs[rows], outs[300], ("normed sum", "residual", "plain norm")):
            assert torch.equal(got, want[:rows]), f"hidden {hidden}: {what} of {rows} rows differs from the same rows among 300"
