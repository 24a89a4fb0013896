"""The generation loop's decisions (no GPU): batching of requests, stop tokens, early ends, limits.
The full loop also runs here over the engine with the plain kernel functions swapped in."""
import numpy as np
import pytest
import torch

import kernel_refs
import plain_gemma2 as plain
import tiny_configs
from rust_deeplearning_b200.config.base import architecture_for
from rust_deeplearning_b200.engine.generate import SequenceState, generate, plan_batches
from rust_deeplearning_b200.engine.step import Engine
from rust_deeplearning_b200.parts.model import Model
from rust_deeplearning_b200.sampling.sampler import SamplingParams, uniform_for
from rust_deeplearning_b200.weights.loader import load_weights
from rust_deeplearning_b200.weights.random_init import write_random_model


def test_plan_batches():
    kw = dict(max_seqs=3, max_tokens=256, page_size=64, max_context=128)
    assert plan_batches([5, 11, 17], 8, **kw) == [[0, 1, 2]]
    assert plan_batches([5, 11, 17, 3], 8, **kw) == [[0, 1, 2], [3]]                 # at most three at once
    assert plan_batches([60, 60, 60], 10, **kw) == [[0, 1], [2]]                      # 128 + 128 fill the cache
    assert plan_batches([1], 1, **kw) == [[0]]
    assert plan_batches([100, 100], 100, **kw) == [[0, 1]]                            # capped by the context: 128 each
    with pytest.raises(ValueError):
        plan_batches([129], 1, **kw)                                                  # prompt longer than the context
    with pytest.raises(ValueError):
        plan_batches([0], 1, **kw)
    with pytest.raises(ValueError):
        plan_batches([100], 8, max_seqs=1, max_tokens=64, page_size=64, max_context=128)


def test_plan_batches_on_requests_drawn_at_random():
    """Every request once and in order; no batch over its limits; a batch ends only where the next request would
    not have fitted."""
    import random
    rnd = random.Random(3)
    for _ in range(300):
        page = rnd.choice([16, 64])
        max_context = rnd.choice([64, 200, 1024])
        max_seqs = rnd.randint(1, 6)
        max_tokens = page * rnd.randint(max_context // page + 1, max_context // page + 40)
        new = rnd.randint(1, 300)
        lens = [rnd.randint(1, max_context) for _ in range(rnd.randint(1, 30))]
        cost = lambda n: -(-min(n + new - 1, max_context) // page) * page
        batches = plan_batches(lens, new, max_seqs=max_seqs, max_tokens=max_tokens, page_size=page, max_context=max_context)
        assert [i for b in batches for i in b] == list(range(len(lens)))
        for k, b in enumerate(batches):
            assert 1 <= len(b) <= max_seqs and sum(cost(lens[i]) for i in b) <= max_tokens
            if k + 1 < len(batches):
                nxt = batches[k + 1][0]
                assert len(b) == max_seqs or sum(cost(lens[i]) for i in b) + cost(lens[nxt]) > max_tokens


def test_sequence_state_decisions():
    s = SequenceState(0, [1, 2, 3], max_new_tokens=3, max_context=100, stop_token_ids=frozenset([9]))
    assert s.accept(4) and s.accept(5) and s.new_tokens == [4, 5] and not s.finished
    assert not s.accept(6) and s.finish_reason == "length" and s.new_tokens == [4, 5, 6] and s.sampled == 3
    s = SequenceState(0, [1], 5, 100, frozenset([9]))
    assert s.accept(4) and not s.accept(9)
    assert s.finish_reason == "stop" and s.new_tokens == [4]                          # the stop token is not kept
    s = SequenceState(0, [1], 5, 100, frozenset([9]), include_stop=True)
    assert not s.accept(9) and s.new_tokens == [9]
    # the context ends the sequence when the sampled token could not be fed back
    s = SequenceState(0, [1, 2, 3], 10, max_context=4, stop_token_ids=frozenset())
    assert s.accept(7)                                                               # 3 + 1 = 4 positions: still fits
    assert not s.accept(8) and s.finish_reason == "context" and s.new_tokens == [7, 8]
    s = SequenceState(0, [1], 1, 100, frozenset())
    assert not s.accept(3) and s.finish_reason == "length"                            # max_new_tokens counts the first token


def test_uniform_numbers():
    xs = [uniform_for(3, r, s) for r in range(50) for s in range(50)]
    assert all(0.0 <= x < 1.0 for x in xs) and len(set(xs)) > 2400
    assert abs(np.mean(xs) - 0.5) < 0.02
    assert uniform_for(3, 1, 2) == uniform_for(3, 1, 2) != uniform_for(4, 1, 2)


def test_sampling_params_are_checked():
    SamplingParams(temperature=0.0)
    for bad in (dict(temperature=-1.0), dict(top_k=0), dict(top_p=0.0), dict(repetition_penalty=0.0)):
        with pytest.raises(ValueError):
            SamplingParams(**bad)
    assert SamplingParams(temperature=0.0).greedy and not SamplingParams().greedy


@pytest.fixture
def engine(tmp_path, monkeypatch):
    kernel_refs.install(monkeypatch)
    cfg, seed = tiny_configs.config("A")
    folder = write_random_model(str(tmp_path / "a"), cfg, seed, "float32")
    arch = architecture_for(cfg)
    spec = arch.build_spec(arch.parse_config(cfg))
    model = Model(spec, load_weights(spec, folder, torch.float32, "cpu"), torch.float32, "cpu")
    return Engine(model, max_tokens=256, max_seqs=3, max_context=64, page_size=8, use_graphs=False), plain.load_folder(folder)


def test_generate_batches_stop_tokens_and_early_ends(engine):
    eng, (cfg, w) = engine
    rng = np.random.default_rng(5)
    prompts = [[int(v) for v in rng.integers(0, 256, size=n)] for n in (5, 11, 17, 2)]     # four requests, three slots
    greedy = SamplingParams(temperature=0.0)
    res = generate(eng, prompts, max_new_tokens=6, sampling=greedy, stop_token_ids=[])
    want = [plain.generate_greedy(cfg, w, p, 6) for p in prompts]
    assert [r.tokens for r in res] == want and all(r.finish_reason == "length" for r in res)
    assert eng.cache.n_free_slots == 3 and all(g.pool.n_free == g.pool.n_pages for g in eng.cache.kv_groups)
    # a stop token ends one request earlier; the others go on
    stop = want[1][2]
    res = generate(eng, prompts, max_new_tokens=6, sampling=greedy, stop_token_ids=[stop])
    for r, full in zip(res, want):
        cut = full.index(stop) if stop in full else None
        assert r.tokens == (full[:cut] if cut is not None else full)
        assert r.finish_reason == ("stop" if cut is not None else "length")
    # a stream callback sees every kept token and can end a request
    seen = []
    res = generate(eng, prompts[:2], max_new_tokens=6, sampling=greedy, stop_token_ids=[],
                   stream=lambda req, tok: (seen.append((req, tok)), req != 0 or len([1 for r, _ in seen if r == 0]) < 2)[1])
    assert res[0].tokens == want[0][:2] and res[1].tokens == want[1]
    assert [t for r, t in seen if r == 1] == want[1]
    assert generate(eng, prompts[:1], max_new_tokens=0, sampling=greedy)[0].tokens == []
    # the context limit ends a sequence
    long_prompt = [int(v) for v in rng.integers(0, 256, size=62)]
    r = generate(eng, [long_prompt], max_new_tokens=10, sampling=greedy, stop_token_ids=[])[0]
    assert r.finish_reason == "context" and len(r.tokens) == 3                       # positions 62, 63 fed; the third cannot be
    assert r.tokens == plain.generate_greedy(cfg, w, long_prompt, 3)


def test_running_one_step_ahead_changes_no_result(engine):
    """The loop queues a step before it has read the tokens of the step before; with that switched off it
    waits for every step.  Same tokens, same reasons, every slot and page given back - also when stop
    tokens end sequences that are already part of a queued step."""
    eng, _ = engine
    rng = np.random.default_rng(8)
    prompts = [[int(v) for v in rng.integers(0, 256, size=n)] for n in (3, 12, 7, 1, 9)]
    for sampling in (SamplingParams(temperature=0.0), SamplingParams(temperature=0.8, top_k=50, seed=3)):
        waited = generate(eng, prompts, max_new_tokens=7, sampling=sampling, stop_token_ids=[], run_ahead=False)
        ahead = generate(eng, prompts, max_new_tokens=7, sampling=sampling, stop_token_ids=[])
        assert [(r.tokens, r.finish_reason) for r in ahead] == [(r.tokens, r.finish_reason) for r in waited]
        # stop at tokens that some sequences produce early, in the middle and as their last token
        stops = {waited[0].tokens[0], waited[1].tokens[3], waited[2].tokens[6]}
        waited = generate(eng, prompts, max_new_tokens=7, sampling=sampling, stop_token_ids=stops, run_ahead=False)
        ahead = generate(eng, prompts, max_new_tokens=7, sampling=sampling, stop_token_ids=stops)
        assert [(r.tokens, r.finish_reason) for r in ahead] == [(r.tokens, r.finish_reason) for r in waited]
        assert any(r.finish_reason == "stop" for r in ahead)
        assert eng.cache.n_free_slots == 3 and all(g.pool.n_free == g.pool.n_pages for g in eng.cache.kv_groups)


def test_seeded_sampling_does_not_depend_on_the_batch(engine):
    eng, _ = engine
    rng = np.random.default_rng(6)
    prompts = [[int(v) for v in rng.integers(0, 256, size=n)] for n in (4, 9, 6)]
    p = SamplingParams(temperature=0.9, top_k=40, top_p=0.95, repetition_penalty=1.1, seed=11)
    together = generate(eng, prompts, max_new_tokens=5, sampling=p, stop_token_ids=[])
    alone = generate(eng, prompts, max_new_tokens=5, sampling=p, stop_token_ids=[], max_batch=1)
    assert [r.tokens for r in together] == [r.tokens for r in alone]
    other = generate(eng, prompts, max_new_tokens=5, sampling=SamplingParams(temperature=0.9, seed=12), stop_token_ids=[])
    assert [r.tokens for r in other] != [r.tokens for r in together]
