"""The engine on a GPU against the plain implementation, in 32-bit and in bfloat16: requests alone
and whole, the last 32 tokens one by one, batches of unequal lengths with slot reuse, long decoding,
first tokens, greedy generation through the entry point."""
import numpy as np
import pytest

import model_helpers as mh
import plain_gemma2 as plain
import tiny_configs

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
NAMES = ["A", "B", "C", "D", "E"]


def vocab(name):
    return tiny_configs.config(name)[0]["vocab_size"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_each_request_alone_and_whole(name, dtype):
    eng = mh.engine(name, dtype)
    for seed, n in ((1, 5), (2, 37), (3, 150)):
        ids = mh.prompt(seed, n, vocab(name))
        slot = eng.new_sequence()
        got = eng.step([slot], [ids], "all")
        mh.assert_logits(got, mh.plain_logits(name, ids), dtype, f"{name} whole n={n}")
        eng.release(slot)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_last_32_tokens_one_by_one(name, dtype):
    eng = mh.engine(name, dtype)
    ids = mh.prompt(4, 90, vocab(name))
    want = mh.plain_logits(name, ids)
    slot = eng.new_sequence()
    mh.assert_logits(eng.step([slot], [ids[:58]], "all"), want[:58], dtype, "prefix")
    for t in range(58, 90):
        mh.assert_logits(eng.step([slot], [[ids[t]]], "all"), want[t:t + 1], dtype, f"{name} position {t}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens(name, dtype):
    """A one-token prompt, then tokens one by one: positions 0, 1, 2, ... each seen for the first time."""
    eng = mh.engine(name, dtype)
    ids = mh.prompt(5, 6, vocab(name))
    want = mh.plain_logits(name, ids)
    slot = eng.new_sequence()
    for t in range(6):
        mh.assert_logits(eng.step([slot], [[ids[t]]], "all"), want[t:t + 1], dtype, f"{name} position {t}")
    # and a two-token prompt
    slot2 = eng.new_sequence()
    mh.assert_logits(eng.step([slot2], [ids[:2]], "all"), want[:2], dtype, "two tokens")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_unequal_batches_shorter_end_earlier_slots_reused(name, dtype):
    """Batches of 3 and 4 requests, one after another on a cache with 4 slots and few pages: each batch's
    prompts in one step, then one token each; shorter requests end earlier; later batches land on the
    slots and pages the earlier ones gave back."""
    eng = mh.engine(name, dtype, max_tokens=6 * 64, max_seqs=4)
    V = vocab(name)
    shapes = [([5, 11, 17], [8, 8, 8]), ([1, 9, 23, 40], [12, 3, 7, 1]), ([64, 2, 33], [2, 30, 5]),
              ([40, 23, 9, 1], [1, 2, 12, 20])]
    for b, (lens, extra) in enumerate(shapes):
        seqs = [mh.prompt(100 + 10 * b + i, n + e, V) for i, (n, e) in enumerate(zip(lens, extra))]
        want = [mh.plain_logits(name, s) for s in seqs]
        slots = [eng.new_sequence() for _ in seqs]
        got = eng.step(slots, [s[:n] for s, n in zip(seqs, lens)], "all")
        mh.assert_logits(got, np.concatenate([w[:n] for w, n in zip(want, lens)]), dtype, f"batch {b} prompts")
        pos = list(lens)
        live = list(range(len(seqs)))
        while live:
            got = eng.step([slots[i] for i in live], [[seqs[i][pos[i]]] for i in live], "last")
            mh.assert_logits(got, np.stack([want[i][pos[i]] for i in live]), dtype, f"batch {b} decode at {pos}")
            for i in live:
                pos[i] += 1
            for i in [i for i in live if pos[i] == len(seqs[i])]:
                eng.release(slots[i])
            live = [i for i in live if pos[i] < len(seqs[i])]
        assert eng.cache.n_free_slots == 4
    if dtype == "bfloat16":
        assert eng.graph_replays > 0      # the captured graphs were the path that ran


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype):
    """Several hundred single-token steps: crosses many pages, wraps the window ring many times."""
    name = "B"
    eng = mh.engine(name, dtype)
    ids = mh.prompt(6, 420, vocab(name))
    want = mh.plain_logits(name, ids)
    slot = eng.new_sequence()
    eng.step([slot], [ids[:3]], [[]])
    for t in range(3, 420):
        got = eng.step([slot], [[ids[t]]], "last")
        if t % 7 == 0 or t > 400:
            mh.assert_logits(got, want[t:t + 1], dtype, f"position {t}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_padding_changes_nothing(dtype):
    """Three sequences run as a padded batch of four (graph shape) give what each gives alone."""
    name = "A"
    eng = mh.engine(name, dtype)
    V = vocab(name)
    seqs = [mh.prompt(200 + i, n, V) for i, n in enumerate((20, 33, 7))]
    slots = [eng.new_sequence() for _ in seqs]
    eng.step(slots, [s[:-3] for s in seqs], [[], [], []])
    for k in (3, 2, 1):
        got = eng.step(slots, [[s[-k]] for s in seqs], "last")
        want = np.stack([mh.plain_logits(name, s)[len(s) - k] for s in seqs])
        mh.assert_logits(got, want, dtype, f"padded decode {k}")


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(name):
    from rust_deeplearning_b200 import Generator
    cfg, w = mh.plain_model(name)
    V = vocab(name)
    lens, new = ([5, 11, 17], 8) if name == "A" else ([1, 9, 23, 40], 12)
    prompts = [mh.prompt(300 + i, n, V) for i, n in enumerate(lens)]
    gen = Generator(mh.loaded_model(name, "float32"), max_batch=4, max_context=128).with_temperature(0.0)
    stops = frozenset(cfg["eos_token_id"] if isinstance(cfg["eos_token_id"], list) else [cfg["eos_token_id"]])
    got = gen.generate_batch(prompts, new)
    for p, g in zip(prompts, got):
        assert g[:len(p)] == p
        assert g[len(p):] == plain.generate_greedy(cfg, w, p, new, stops)
    # one by one gives the same tokens as the batch
    for p, g in zip(prompts, got):
        assert gen.generate(p, new) == g
    # The bfloat16 path: its batch and its singles agree, and every token agrees with the 32-bit path's as long
    # as the plain logits' margin between the best and the second best token exceeds the bfloat16 tolerance
    # (after a token chosen inside that margin the sequences may part ways, so the comparison stops there).
    gen16 = Generator(mh.loaded_model(name, "bfloat16"), max_batch=4, max_context=128).with_temperature(0.0)
    got16 = gen16.generate_batch(prompts, new)
    compared = 0
    for p, g32, g16 in zip(prompts, got, got16):
        assert g16[:len(p)] == p
        assert gen16.generate(p, new) == g16
        for k in range(len(p), len(g32)):
            logits = plain.forward(cfg, w, g32[:k])[-1]
            top2 = np.sort(logits)[-2:]
            if top2[1] - top2[0] <= 2 * mh.tolerance("bfloat16", logits[None]):
                break
            assert k < len(g16) and g16[k] == g32[k], f"bfloat16 token {k - len(p)} of a prompt of {len(p)} differs"
            compared += 1
    assert compared > 0


@pytest.mark.parametrize("options", [dict(), dict(top_k=20), dict(top_p=0.9), dict(top_k=50, top_p=0.95),
                                     dict(repetition_penalty=1.2), dict(top_k=5, repetition_penalty=1.5)])
def test_temperature_generation_equals_the_plain_sampler(options):
    """T = 0.8, seeded: the tokens of the BASELINE workload of tiny B (prompts of 1, 9, 23 and 40 tokens, 12 new)
    equal what the plain implementation samples from its own logits with the same uniform numbers
    (seed, request index, step) - as a batch, and one request at a time.  With a repetition penalty a token
    that came n times (in the prompt or since) is penalised n times, as the reference's loop over the history does."""
    from rust_deeplearning_b200 import Generator
    from rust_deeplearning_b200.sampling.sampler import uniform_for
    name, seed, new = "B", 7, 12
    cfg, w = mh.plain_model(name)
    V = vocab(name)
    prompts = [mh.prompt(400 + i, n, V) for i, n in enumerate((1, 9, 23, 40))]
    want = []
    for i, p in enumerate(prompts):
        tokens = list(p)
        for step in range(new):
            logits = plain.forward(cfg, w, tokens)[-1].astype(np.float32)
            tokens.append(plain.sample_token(logits, tokens, uniform_for(seed, i, step), temperature=0.8, **options))
        want.append(tokens)
    gen = (Generator(mh.loaded_model(name, "float32"), max_batch=4, max_context=128)
           .with_temperature(0.8).with_seed(seed).with_stop_tokens([])
           .with_top_k(options.get("top_k")).with_top_p(options.get("top_p"))
           .with_repetition_penalty(options.get("repetition_penalty")))
    assert gen.generate_batch(prompts, new) == want
    # one at a time: request i alone is request 0 of its own call, so its stream is keyed by 0
    alone = gen.generate(prompts[0], new)
    assert alone == want[0]


@pytest.mark.parametrize("name", ["B"])
def test_seeded_temperature_sampling_is_batch_independent(name):
    from rust_deeplearning_b200 import Generator
    V = vocab(name)
    prompts = [mh.prompt(400 + i, n, V) for i, n in enumerate((1, 9, 23, 40))]
    gen = (Generator(mh.loaded_model(name, "float32"), max_batch=4, max_context=128)
           .with_temperature(0.8).with_seed(7).with_stop_tokens([]))
    a = gen.generate_batch(prompts, 12)
    b = gen.generate_batch(prompts, 12)
    assert a == b                                            # reproducible
    assert all(len(g) == len(p) + 12 for p, g in zip(prompts, a))
    gen2 = (Generator(mh.loaded_model(name, "float32"), max_batch=2, max_context=128)
            .with_temperature(0.8).with_seed(7).with_stop_tokens([]))
    assert gen2.generate_batch(prompts, 12) == a             # two batches of two: same tokens per request
    assert gen.with_seed(8).generate_batch(prompts, 12) != a
