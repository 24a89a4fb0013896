"""The engine's host logic (packing, paging, rings, slots, schedules) on a machine without a GPU:
the CUDA entry points are replaced by the plain functions of tests/kernel_refs.py, everything
above them is the product's code.  Logits are compared with the plain implementation."""
import numpy as np
import pytest
import torch

import kernel_refs
import plain_gemma2 as plain
import tiny_configs
from rust_deeplearning_b200.config.base import architecture_for
from rust_deeplearning_b200.engine.step import Engine
from rust_deeplearning_b200.parts.model import Model
from rust_deeplearning_b200.weights.loader import load_weights
from rust_deeplearning_b200.weights.random_init import write_random_model

TOL = 2e-5   # float32 activations between float64 kernels


def build(tmp_path, name, monkeypatch, page_size=4, max_tokens=4096, max_seqs=None):
    kernel_refs.install(monkeypatch)
    cfg, seed = tiny_configs.config(name)
    folder = str(tmp_path / f"tiny_{name}")
    write_random_model(folder, cfg, seed, "float32")
    arch = architecture_for(cfg)
    spec = arch.build_spec(arch.parse_config(cfg))
    model = Model(spec, load_weights(spec, folder, torch.float32, "cpu"), torch.float32, "cpu")
    engine = Engine(model, max_tokens=max_tokens, max_seqs=max_seqs, page_size=page_size, use_graphs=False)
    pcfg, pw = plain.load_folder(folder)
    return engine, pcfg, pw


def prompt(rng, n, vocab):
    return [int(v) for v in rng.integers(0, vocab, size=n)]


def close(got, want):
    got = got.detach().cpu().double().numpy()
    assert got.shape == want.shape
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= TOL, np.abs(got - want).max()


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompt_equals_plain(tmp_path, monkeypatch, name):
    engine, cfg, w = build(tmp_path, name, monkeypatch)
    rng = np.random.default_rng(1)
    ids = prompt(rng, 37, cfg["vocab_size"])          # longer than both windows
    slot = engine.new_sequence()
    logits = engine.step([slot], [ids], "all")
    close(logits, plain.forward(cfg, w, ids))


@pytest.mark.parametrize("name", ["A", "B"])
def test_token_by_token_and_chunks_equal_plain(tmp_path, monkeypatch, name):
    engine, cfg, w = build(tmp_path, name, monkeypatch)
    rng = np.random.default_rng(2)
    ids = prompt(rng, 45, cfg["vocab_size"])
    want = plain.forward(cfg, w, ids)
    # a prefix whole, then one by one
    slot = engine.new_sequence()
    close(engine.step([slot], [ids[:13]], "all"), want[:13])
    for t in range(13, 45):
        close(engine.step([slot], [[ids[t]]], "all"), want[t:t + 1])
    engine.release(slot)
    # the same in three chunks: a chunk after an existing prefix reads cache and new rows
    slot = engine.new_sequence()
    close(engine.step([slot], [ids[:7]], "all"), want[:7])
    close(engine.step([slot], [ids[7:30]], "all"), want[7:30])
    close(engine.step([slot], [ids[30:]], "all"), want[30:])


@pytest.mark.parametrize("name", ["A", "B"])
def test_unequal_batches_and_slot_reuse(tmp_path, monkeypatch, name):
    engine, cfg, w = build(tmp_path, name, monkeypatch, max_tokens=256, max_seqs=4)
    rng = np.random.default_rng(3)
    V = cfg["vocab_size"]
    for round_ in range(3):                      # one batch after another on the same small cache
        lens = [1, 9, 23, 40] if round_ % 2 == 0 else [17, 5, 11]
        extra = [3, 12, 6, 1]
        seqs = [prompt(rng, n + e, V) for n, e in zip(lens, extra)]
        want = [plain.forward(cfg, w, s) for s in seqs]
        slots = [engine.new_sequence() for _ in seqs]
        got = engine.step(slots, [s[:n] for s, n in zip(seqs, lens)], "all")
        close(got, np.concatenate([wv[:n] for wv, n in zip(want, lens)]))
        pos = list(lens)
        live = list(range(len(seqs)))
        while live:
            got = engine.step([slots[i] for i in live], [[seqs[i][pos[i]]] for i in live], "last")
            close(got, np.stack([want[i][pos[i]] for i in live]))
            for i in live:
                pos[i] += 1
            for i in [i for i in live if pos[i] == len(seqs[i])]:
                engine.release(slots[i])         # shorter requests end earlier
            live = [i for i in live if pos[i] < len(seqs[i])]
        assert engine.cache.n_free_slots == 4
        assert all(g.pool.n_free == g.pool.n_pages for g in engine.cache.kv_groups)


def test_wanted_places_and_errors(tmp_path, monkeypatch):
    engine, cfg, w = build(tmp_path, "A", monkeypatch)
    from rust_deeplearning_b200.engine.step import StepError
    rng = np.random.default_rng(4)
    a, b = prompt(rng, 6, 256), prompt(rng, 11, 256)
    s0, s1 = engine.new_sequence(), engine.new_sequence()
    got = engine.step([s0, s1], [a, b], [[0, 5], []])
    close(got, plain.forward(cfg, w, a)[[0, 5]])
    assert engine.length(s0) == 6 and engine.length(s1) == 11
    got = engine.step([s1, s0], [[3], [4]], [[0], []])
    close(got, plain.forward(cfg, w, b + [3])[-1:])
    with pytest.raises(StepError):
        engine.step([s0], [[256]])
    with pytest.raises(StepError):
        engine.step([s0], [[]])
    with pytest.raises(StepError):
        engine.step([s0], [[1.5]])                # no whole number: refused, not cut down to 1
    with pytest.raises(StepError):
        engine.step([s0], [[True]])
    with pytest.raises(StepError):
        engine.step([s0], [[3, 4]], [[0.5]])
    assert engine.length(s0) == 7                 # failed steps changed nothing


def test_a_walk_of_valid_and_invalid_steps_drawn_at_random(tmp_path, monkeypatch):
    """Four slots on a cache of 160 rows: sequences begin and are given back, steps bring 1 to 17 tokens for any
    subset of them and want any places, and about a third of the steps are wrong in one way (an empty list, an id
    outside the vocabulary or no whole number, a slot twice or not in use, a wanted place outside, more tokens than
    the context or the cache holds, tokens for too few sequences).  A wrong step raises the engine's own error and
    changes no length; a right one gives the plain implementation's logits, whatever came before."""
    import random
    from rust_deeplearning_b200.cache.cache import CacheError
    from rust_deeplearning_b200.engine.step import StepError
    engine, cfg, w = build(tmp_path, "A", monkeypatch, page_size=4, max_tokens=160, max_seqs=4)
    V = cfg["vocab_size"]
    rnd = random.Random(5)
    live, checked, refused = {}, 0, 0          # slot -> the tokens it holds
    for _ in range(90):
        kind = rnd.random()
        if kind < 0.15 and len(live) < 4:
            live[engine.new_sequence()] = []
            continue
        if kind < 0.25 and live:
            slot = rnd.choice(list(live))
            engine.release(slot)
            del live[slot]
            continue
        if kind < 0.30:
            with pytest.raises((StepError, CacheError)):
                if rnd.random() < 0.5:
                    engine.release(rnd.choice([-1, 99] + [s for s in range(4) if s not in live]))
                else:
                    for _ in range(5 - len(live)):
                        live[engine.new_sequence()] = []
            refused += 1
            continue
        if not live:
            continue
        slots = rnd.sample(list(live), rnd.randint(1, len(live)))
        toks = [[rnd.randrange(V) for _ in range(rnd.choice([1, 1, 2, 5, 17]))] for _ in slots]
        want = rnd.choice(["last", "all", None])
        if want is None:
            want = [sorted(rnd.sample(range(len(t)), rnd.randint(0, len(t)))) for t in toks]
        before = {s: engine.length(s) for s in live}
        if rnd.random() < 0.35:
            k = rnd.randrange(9)
            if k == 0: toks[0] = []
            elif k == 1: toks[0] = [V + rnd.randrange(3)]
            elif k == 2: toks[0] = [-1]
            elif k == 3: slots, toks = slots + [slots[0]], toks + [toks[0]]
            elif k == 4: slots[0] = rnd.choice([-1, 99] + [s for s in range(4) if s not in live])
            elif k == 5: want = [[len(t)] for t in toks]
            elif k == 6: toks[0] = [rnd.randrange(V) for _ in range(600)]
            elif k == 7: toks = toks[:-1] if len(toks) > 1 else toks + [[1]]
            elif k == 8: toks[0] = [1.5]
            if k in (5, 7) and not isinstance(want, str) and len(want) != len(toks):
                want = "last"
            with pytest.raises((StepError, CacheError)):
                engine.step(slots, toks, want)
            assert {s: engine.length(s) for s in live} == before, f"a refused step (kind {k}) changed a length"
            refused += 1
            continue
        try:
            got = engine.step(slots, toks, want)
        except CacheError:                      # the cache is full: nothing may have changed
            assert {s: engine.length(s) for s in live} == before
            refused += 1
            continue
        places = [[len(t) - 1] for t in toks] if want == "last" else ([list(range(len(t))) for t in toks] if want == "all" else want)
        rows = []
        for slot, t, ws in zip(slots, toks, places):
            if ws:
                rows += list(plain.forward(cfg, w, live[slot] + t)[[len(live[slot]) + i for i in ws]])
            live[slot] = live[slot] + t
        if rows:
            close(got, np.stack(rows))
            checked += 1
    assert checked > 20 and refused > 10, (checked, refused)


def test_a_run_that_reads_another_runs_ring_sees_the_rows_of_earlier_steps(tmp_path, monkeypatch):
    """Schedule: layer 0 with a window of 8 keeps a ring of 3 pages of 4 rows; layer 1 reads layer 0's keys and
    values.  A portion of 10 tokens on a prefix of 9 lands on ring rows that the portion's early queries still
    read in layer 1, so layer 0's write has to wait until layer 1 has run.  Whole, in portions and token by
    token must agree (the whole prompt reads no ring at all)."""
    import dataclasses
    from rust_deeplearning_b200.parts.spec import ScheduleEntry
    kernel_refs.install(monkeypatch)
    cfg, seed = tiny_configs.config("A")
    cfg["layer_types"] = ["sliding_attention", "sliding_attention"]
    folder = str(tmp_path / "shared")
    write_random_model(folder, cfg, seed, "float32")
    arch = architecture_for(cfg)
    spec = arch.build_spec(arch.parse_config(cfg))
    spec = dataclasses.replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1, reads_cache_of=0)))
    model = Model(spec, load_weights(spec, folder, torch.float32, "cpu"), torch.float32, "cpu")
    engine = Engine(model, max_tokens=4096, page_size=4, use_graphs=False)
    assert engine.cache.kv_groups[0].is_ring and engine.cache.kv_groups[0].ring_pages == 3
    rng = np.random.default_rng(9)
    ids = prompt(rng, 40, cfg["vocab_size"])
    slot = engine.new_sequence()
    whole = engine.step([slot], [ids], "all").double().numpy()
    engine.release(slot)
    slot = engine.new_sequence()
    parts = [engine.step([slot], [ids[a:b]], "all") for a, b in ((0, 9), (9, 19), (19, 20), (20, 40))]
    close(torch.cat(parts), whole)
    engine.release(slot)
    slot = engine.new_sequence()
    close(torch.cat([engine.step([slot], [[t]], "all") for t in ids]), whole)
