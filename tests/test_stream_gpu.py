"""The residual stream's split form of the norms around few-row products (`parts/norm.py`): the same chain
of branches run with every offer taken, with single offers declined at each place, with another norm than
the announced one, and with the stream's value asked for in between - always against the float64 formulas.
The split form is an offer between parts; whatever a part declines must come out the same."""
import pytest
import torch

import kernel_refs as ref
from rust_deeplearning_b200.kernels import ops
from rust_deeplearning_b200.parts.norm import ResidualStream, RMSNorm

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
BF16 = torch.bfloat16


def rnd(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(DEV)


class Chain:
    """Three branches on a stream of `rows` x `width`: x -> (W_in, W_out) -> post norm -> add, each followed by
    a norm; the last norm's rows (a selection) go into a head product."""

    def __init__(self, rows, width, inner):
        self.rows, self.width = rows, width
        self.h0 = rnd((rows, width), torch.float32, 1, 2.0)
        self.pre = [RMSNorm(rnd((width,), BF16, 10 + i, 0.5), 1e-6, 1.0) for i in range(4)]      # pre[3]: the final norm
        self.post = [RMSNorm(rnd((width,), torch.float32 if i == 1 else BF16, 20 + i, 0.5), 1e-5, 1.0) for i in range(3)]
        self.w_in = [rnd((inner, width), BF16, 30 + i, 0.1) for i in range(3)]
        self.w_out = [rnd((width, inner), BF16, 40 + i, 0.1) for i in range(3)]
        self.w_head = rnd((200, width), BF16, 50, 0.1)
        self.pick = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)

    def reference(self):
        h = self.h0.double()
        p = lambda n: (n.weight, n.eps, n.offset)
        for i in range(3):
            x = ref._rms(h, p(self.pre[i]))
            y = (x @ self.w_in[i].double().t()) @ self.w_out[i].double().t()
            h = h + ref._rms(y, p(self.post[i]))
        logits = ref._rms(h, p(self.pre[3]))[self.pick.long()] @ self.w_head.double().t()
        return h, logits

    def run(self, takes, delivers, wrong_norm_at=None, value_at=None):
        """takes[i]: consumer i (0..2 the branches' first products, 3 the head) accepts deferred rows;
        delivers[i]: branch i's last product uses the sink.  Returns (stream value, logits, what each consumer got)."""
        stream = ResidualStream(self.h0.clone())
        got = []
        for i in range(3):
            nxt = self.pre[i + 1]
            announce = delivers[i] and takes[i + 1]
            x = stream.normed(self.pre[i], BF16, deferred_ok=takes[i], upcoming=nxt if announce else None)
            got.append(type(x).__name__)
            sink = stream.branch_sink(self.post[i], nxt) if announce else None
            mid = ops.linear(x, self.w_in[i])
            y = ops.linear_branch(mid, self.w_out[i], sink) if sink is not None else ops.linear(mid, self.w_out[i])
            stream.add(y, self.post[i])
            if value_at == i:
                stream.value()
            if wrong_norm_at == i:
                # somebody asks for another norm than the one announced: plain kernels, same numbers
                other = RMSNorm(self.pre[0].weight, 1e-6, 1.0)
                want = ref._rms(stream_value_after(self, i), (other.weight, other.eps, other.offset))
                close(stream.normed(other, BF16, deferred_ok=True), want, "another norm than the announced one")
        n = stream.normed_rows(self.pre[3], self.pick, BF16, deferred_ok=takes[3])
        got.append(type(n).__name__)
        logits = ops.linear(n, self.w_head, out_dtype=torch.float32)
        return stream.value(), logits, got


def stream_value_after(chain, i):
    h = chain.h0.double()
    p = lambda n: (n.weight, n.eps, n.offset)
    for j in range(i + 1):
        x = ref._rms(h, p(chain.pre[j]))
        h = h + ref._rms((x @ chain.w_in[j].double().t()) @ chain.w_out[j].double().t(), p(chain.post[j]))
    return h


def close(got, want, what, rel=0.02):
    got, want = got.double().cpu(), want.double().cpu()
    assert got.shape == want.shape, (what, got.shape, want.shape)
    scale = want.abs().max().item()
    err = (got - want).abs().max().item()
    assert err <= rel * scale, f"{what}: error {err:.3e} > {rel * scale:.3e}"


@pytest.mark.parametrize("rows,width,inner", [(5, 96, 64), (8, 2304, 256), (1, 1000, 40)])
def test_every_offer_taken_and_every_single_offer_declined(rows, width, inner):
    chain = Chain(rows, width, inner)
    h_ref, logits_ref = chain.reference()
    all_yes = ([True] * 4, [True] * 3)
    h, logits, got = chain.run(*all_yes)
    assert got == ["Tensor", "DeferredRows", "DeferredRows", "DeferredRows"], got
    close(h, h_ref, "stream, all offers taken", rel=0.01)
    close(logits, logits_ref, "logits, all offers taken")
    for k in range(7):
        takes, delivers = [True] * 4, [True] * 3
        (takes if k < 4 else delivers)[k if k < 4 else k - 4] = False
        h, logits, got = chain.run(takes, delivers)
        close(h, h_ref, f"stream, offer {k} declined", rel=0.01)
        close(logits, logits_ref, f"logits, offer {k} declined")
        want = ["Tensor"] + ["DeferredRows" if takes[i + 1] and delivers[i] else "Tensor" for i in range(3)]
        assert got == want, (k, got, want)
    h, logits, got = chain.run([False] * 4, [False] * 3)
    assert got == ["Tensor"] * 4
    close(h, h_ref, "stream, no offers", rel=0.01)
    close(logits, logits_ref, "logits, no offers")


@pytest.mark.parametrize("where", [0, 1, 2])
def test_the_value_or_another_norm_asked_for_in_between(where):
    chain = Chain(5, 96, 64)
    h_ref, logits_ref = chain.reference()
    h, logits, _ = chain.run([True] * 4, [True] * 3, value_at=where)
    close(h, h_ref, "stream", rel=0.01)
    close(logits, logits_ref, "logits")
    if where < 2:
        chain.run([True] * 4, [True] * 3, wrong_norm_at=where)


def test_many_rows_and_float32_streams_use_the_norm_kernels():
    for rows, dtype in ((9, BF16), (5, torch.float32)):
        chain = Chain(rows, 96, 64)
        if dtype is torch.float32:
            for name in ("w_in", "w_out"):
                setattr(chain, name, [w.float() for w in getattr(chain, name)])
        stream = ResidualStream(chain.h0.clone())
        x = stream.normed(chain.pre[0], dtype, deferred_ok=True, upcoming=chain.pre[1])
        assert isinstance(x, torch.Tensor) and stream.branch_sink(chain.post[0], chain.pre[1]) is None


def test_rows_handed_out_must_be_used():
    chain = Chain(4, 96, 64)
    stream = ResidualStream(chain.h0.clone())
    x = stream.normed(chain.pre[0], BF16, deferred_ok=True, upcoming=chain.pre[1])
    sink = stream.branch_sink(chain.post[0], chain.pre[1])
    stream.add(ops.linear_branch(ops.linear(x, chain.w_in[0]), chain.w_out[0], sink), chain.post[0])
    rows = stream.normed(chain.pre[1], BF16, deferred_ok=True)
    assert isinstance(rows, ops.DeferredRows)
    with pytest.raises(RuntimeError, match="must go into a product"):
        stream.value()
    close(rows.materialise(), ref._rms(stream_value_after(chain, 0), (chain.pre[1].weight, chain.pre[1].eps, chain.pre[1].offset)), "materialised")
    close(stream.value(), stream_value_after(chain, 0), "stream", rel=0.01)


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_the_engine_decodes_without_norm_kernels(name, monkeypatch):
    """Single-token steps of a real model: with the split form a step launches fewer kernels (no norm kernel between a
    branch's last product and the next part's first), and the logits agree with the plain implementation as they do
    through the norm kernels."""
    import model_helpers as mh
    import tiny_configs
    from rust_deeplearning_b200.kernels import library
    cfg = tiny_configs.config(name)[0]
    ids = mh.prompt(800, 40, cfg["vocab_size"])
    want = mh.plain_logits(name, ids)
    counts = {}
    for split in (True, False):
        monkeypatch.setattr(ops, "DEFERRED_NORMS", split)
        eng = mh.engine(name, "bfloat16", use_graphs=False)
        slot = eng.new_sequence()
        eng.step([slot], [ids[:30]], [[]])
        rows = []
        before = library.launch_count
        for t in range(30, 40):
            rows.append(eng.step([slot], [[ids[t]]], "last").clone())
        counts[split] = library.launch_count - before
        mh.assert_logits(torch.cat(rows), want[30:40], "bfloat16", f"{name}, split form {split}")
        eng.release(slot)
    assert counts[True] < counts[False], counts


@pytest.mark.parametrize("name", ["A", "D"])
def test_seven_sequences_decode_together(name):
    """Five to eight rows take the 16-row operand (up to four share one fragment): seven sequences of unequal length,
    single-token steps through the captured graph, every logit against the plain implementation."""
    import numpy as np
    import model_helpers as mh
    import tiny_configs
    cfg = tiny_configs.config(name)[0]
    V = cfg["vocab_size"]
    seqs = [mh.prompt(810 + i, 12 + 5 * i, V) for i in range(7)]
    want = [mh.plain_logits(name, s) for s in seqs]
    eng = mh.engine(name, "bfloat16", max_seqs=8)
    slots = [eng.new_sequence() for _ in seqs]
    cut = [len(s) - 6 for s in seqs]
    eng.step(slots, [s[:c] for s, c in zip(seqs, cut)], [[] for _ in seqs])
    for k in range(6):
        got = eng.step(slots, [[s[c + k]] for s, c in zip(seqs, cut)], "last")
        mh.assert_logits(got, np.stack([w[c + k] for w, c in zip(want, cut)]), "bfloat16", f"{name}, step {k}")
    assert eng.graph_replays > 0
