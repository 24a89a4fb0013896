"""Generation workloads drawn at random (seeded): 1 to 11 requests with prompts of 1 to 49 tokens, 1 to 13 new
tokens, batches of at most 1 to 5 requests one after another, greedy or seeded temperature sampling with top-k,
top-p and a repetition penalty, a stop token that the first request is known to produce, and a context that
some requests fill before they have their tokens - the tokens of
`Generator.generate_batch` in float32 against the plain implementation's loop, which re-runs the whole sequence
for every token and samples with the same uniform numbers."""
import numpy as np
import pytest

import model_helpers as mh
import plain_gemma2 as plain

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("first", range(0, 40, 8))
def test_generation_workloads_drawn_at_random(first):
    from rust_deeplearning_b200 import Generator
    from rust_deeplearning_b200.sampling.sampler import uniform_for
    for case in range(first, first + 8):
        rng = np.random.default_rng(case)
        name = ["A", "B", "D", "C"][case % 4]
        cfg, w = mh.plain_model(name)
        n_requests = int(rng.integers(1, 12))
        lengths = [int(v) for v in rng.integers(1, 50, size=n_requests)]
        new, max_batch = int(rng.integers(1, 14)), int(rng.integers(1, 6))
        prompts = [mh.prompt(5000 + 20 * case + i, n, cfg["vocab_size"]) for i, n in enumerate(lengths)]
        temperature, seed = float(rng.choice([0.0, 0.8, 0.8])), int(rng.integers(0, 1000))
        options = {}
        if temperature and rng.integers(0, 2):
            options["top_k"] = int(rng.choice([1, 5, 40]))
        if temperature and rng.integers(0, 2):
            options["top_p"] = float(rng.choice([0.5, 0.9]))
        if temperature and rng.integers(0, 2):
            options["repetition_penalty"] = 1.2
        max_context = int(rng.integers(max(lengths), max(lengths) + new + 3))     # some requests run out of context
        greedy = plain.generate_greedy(cfg, w, prompts[0], new, ())
        stops = frozenset([greedy[len(greedy) // 2]] if rng.integers(0, 2) else [])
        want = []
        for i, p in enumerate(prompts):
            tokens = list(p)
            for step in range(new):
                logits = plain.forward(cfg, w, tokens)[-1].astype(np.float32)
                t = plain.sample_token(logits, tokens, uniform_for(seed, i, step), temperature=temperature, **options)
                if t in stops:
                    break
                tokens.append(t)
                if len(tokens) > max_context:       # it was sampled from the last position; it cannot be fed back
                    break
            want.append(tokens)
        gen = (Generator(mh.loaded_model(name, "float32"), max_batch=max_batch, max_context=max_context)
               .with_temperature(temperature).with_seed(seed).with_stop_tokens(stops)
               .with_top_k(options.get("top_k")).with_top_p(options.get("top_p"))
               .with_repetition_penalty(options.get("repetition_penalty")))
        got = gen.generate_batch(prompts, new)
        assert got == want, (f"case {case}: {name}, prompts of {lengths}, {new} new, context {max_context}, batches of {max_batch}, T {temperature}, "
                             f"{options}, stops {set(stops)}")
