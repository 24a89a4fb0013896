"""The plain implementation's own invariants and its sampling functions (no GPU).  The sampling
cases mirror the reference's unit tests, rustml/nlp/main/src/core/sampling.rs:131-231."""
import math

import numpy as np
import pytest

import plain_gemma2 as plain
import tiny_configs
from rust_deeplearning_b200.weights.random_init import write_random_model


def test_parts():
    x = np.array([[3.0, 4.0]])
    assert np.allclose(plain.rms_norm(x, np.zeros(2), 0.0, offset=1.0), x / math.sqrt(12.5))
    assert np.allclose(plain.rms_norm(x, np.ones(2), 0.0, offset=1.0), 2 * x / math.sqrt(12.5))   # (1 + w)
    assert plain.gelu_tanh(np.array([0.0]))[0] == 0.0
    assert abs(plain.gelu_tanh(np.array([1.0]))[0] - 0.841192) < 1e-5
    cos, sin = plain.rope_tables(8, 5, 10000.0)
    assert np.allclose(cos[0], 1) and np.allclose(sin[0], 0) and cos.shape == (5, 4)
    assert np.allclose(cos[3, 1], math.cos(3 * 10000.0 ** (-2 / 8)))
    v = np.arange(16, dtype=float).reshape(1, 2, 8)
    r = plain.rope_apply(np.repeat(v, 5, axis=0), cos, sin)
    assert np.allclose(r[0], v[0])                                                # position 0 is the identity
    assert np.allclose(np.linalg.norm(r, axis=-1), np.linalg.norm(v, axis=-1))    # a rotation
    assert np.allclose(r[2, 0, 0], v[0, 0, 0] * cos[2, 0] - v[0, 0, 4] * sin[2, 0])     # pairs (i, i + d/2)
    m = plain.attention_mask(5, 2)
    assert m.tolist() == [[True, False, False, False, False], [True, True, False, False, False],
                          [False, True, True, False, False], [False, False, True, True, False],
                          [False, False, False, True, True]]
    assert (plain.attention_mask(5, None) == np.tril(np.ones((5, 5), bool))).all()
    assert plain.layer_window({"sliding_window": 8}, 0) == 8 and plain.layer_window({"sliding_window": 8}, 1) is None


@pytest.fixture(scope="module")
def model_b(tmp_path_factory):
    cfg, seed = tiny_configs.config("B")
    return plain.load_folder(write_random_model(str(tmp_path_factory.mktemp("plain") / "b"), cfg, seed, "float32"))


def test_forward_is_causal_windowed_and_capped(model_b):
    cfg, w = model_b
    rng = np.random.default_rng(0)
    ids = [int(v) for v in rng.integers(0, cfg["vocab_size"], size=40)]
    full = plain.forward(cfg, w, ids)
    assert full.shape == (40, cfg["vocab_size"]) and np.abs(full).max() < cfg["final_logit_softcapping"]
    assert np.allclose(plain.forward(cfg, w, ids[:23]), full[:23], atol=1e-12)          # later tokens change nothing
    other = list(ids)
    other[0] = (other[0] + 1) % cfg["vocab_size"]
    changed = plain.forward(cfg, w, other)
    assert not np.allclose(changed[10], full[10])                                        # global layers see position 0
    wide = dict(cfg, sliding_window=1000)
    assert not np.allclose(plain.forward(wide, w, ids)[39], full[39])                   # the window of 16 matters
    assert np.allclose(plain.forward(wide, w, ids)[:16], full[:16], atol=1e-12)         # but not within its first 16
    uncapped = dict(cfg, final_logit_softcapping=None)
    z = plain.forward(uncapped, w, ids)
    assert np.allclose(15.0 * np.tanh(z / 15.0), full, atol=1e-12)
    with pytest.raises(IndexError):
        plain.forward(cfg, w, [cfg["vocab_size"]])
    with pytest.raises(ValueError):
        plain.forward(dict(cfg, max_position_embeddings=8), w, ids)


def test_sampling_functions():
    assert plain.argmax([1.0, 5.0, 3.0, 5.0]) == 1                                      # first maximum wins
    p = plain.apply_repetition_penalty([2.0, -2.0, 1.0], [0, 1], 2.0)
    assert p.tolist() == [1.0, -4.0, 1.0]
    assert plain.apply_repetition_penalty([2.0], [0, 0], 2.0).tolist() == [0.5]          # once per occurrence
    k = plain.apply_top_k([1.0, 5.0, 3.0, 2.0, 4.0], 2)
    assert [v > -np.inf for v in k] == [False, True, False, False, True]
    assert (plain.apply_top_k([1.0, 2.0], 5) == np.array([1.0, 2.0], np.float32)).all()  # k >= len: unchanged
    ties = plain.apply_top_k([3.0, 3.0, 1.0], 1)
    assert [v > -np.inf for v in ties] == [True, True, False]                            # ties with the k-th are kept
    tp = plain.apply_top_p([10.0, 0.0, 0.0, 0.0], 0.5)
    assert [v > -np.inf for v in tp] == [True, False, False, False]
    tp = plain.apply_top_p([1.0, 1.0, 1.0, 1.0], 0.6)
    assert sum(v > -np.inf for v in tp) == 3                                             # the crossing token is kept
    assert (plain.apply_top_p([1.0, 2.0], 1.0) == np.array([1.0, 2.0], np.float32)).all()
    assert plain.sample_categorical([0.0, 100.0, 0.0], 0.3) == 1                         # degenerate distribution
    assert plain.sample_categorical([0.0, 0.0], 0.49) == 0 and plain.sample_categorical([0.0, 0.0], 0.51) == 1
    counts = np.bincount([plain.sample_categorical([0.0, 0.0, 0.0, 0.0], (i + 0.5) / 400) for i in range(400)])
    assert counts.tolist() == [100, 100, 100, 100]                                       # uniform
    assert plain.sample_token([1.0, 3.0, 2.0], [], 0.9, temperature=0.0) == 1
    assert plain.sample_token([1.0, 3.0, 2.0], [], 0.9999, temperature=1.0, top_k=1) == 1
