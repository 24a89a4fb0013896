"""Shared by the GPU tests: tiny model folders, engines on them, the plain logits, tolerances."""
import functools
import os
import tempfile

import numpy as np
import torch

import plain_gemma2 as plain
import tiny_configs

_TMP = None


def tmp_root():
    global _TMP
    if _TMP is None:
        _TMP = tempfile.TemporaryDirectory(prefix="rdl_tests_")
    return _TMP.name


@functools.lru_cache(maxsize=None)
def model_folder(name: str) -> str:
    """A random model folder for tiny configuration `name`, stored in bfloat16 so that the
    32-bit path, the bfloat16 path and the plain implementation all see the same weights."""
    from rust_deeplearning_b200 import write_random_model
    cfg, seed = tiny_configs.config(name)
    folder = os.path.join(tmp_root(), f"tiny_{name}")
    write_random_model(folder, cfg, seed, "bfloat16")
    return folder


@functools.lru_cache(maxsize=None)
def plain_model(name: str):
    return plain.load_folder(model_folder(name))


@functools.lru_cache(maxsize=None)
def loaded_model(name: str, dtype: str):
    from rust_deeplearning_b200 import load_model
    return load_model(model_folder(name), dtype, "cuda:0")


def engine(name: str, dtype: str, **kw):
    from rust_deeplearning_b200 import Engine
    kw.setdefault("max_tokens", 4096)
    return Engine(loaded_model(name, dtype), **kw)


_PLAIN_CACHE = {}


def plain_logits(name: str, ids):
    key = (name, tuple(ids))
    if key not in _PLAIN_CACHE:
        cfg, w = plain_model(name)
        _PLAIN_CACHE[key] = plain.forward(cfg, w, list(ids))
    return _PLAIN_CACHE[key]


def prompt(seed: int, n: int, vocab: int):
    rng = np.random.default_rng(seed)
    return [int(v) for v in rng.integers(0, vocab, size=n)]


def tolerance(dtype: str, want: np.ndarray, bf16_fraction: float = 0.02) -> float:
    """Set from what the tests observe (conftest prints the largest error over the largest logit at the end
    of a session).  float32: 2e-5 of the largest logit, at least 2e-5 (observed: 2e-6).  bfloat16: 2 % of the
    largest logit plus a small absolute floor (observed on the tiny configurations: 1.1 %; the tests at
    real layer sizes, where thousands of terms average the roundings out, observe 0.2 % and pass 0.5 %)."""
    scale = float(np.abs(want).max())
    return 2e-5 * max(1.0, scale) if dtype == "float32" else bf16_fraction * scale + 1e-3


OBSERVED = {}    # dtype -> largest (error / largest logit) seen by assert_logits in this session; conftest prints it


def assert_logits(got: torch.Tensor, want: np.ndarray, dtype: str, what="", bf16_fraction: float = 0.02):
    got = got.detach().float().cpu().double().numpy()
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    err = np.abs(got - want)
    tol = tolerance(dtype, want, bf16_fraction)
    if err.size:
        OBSERVED[dtype] = max(OBSERVED.get(dtype, 0.0), float(err.max()) / max(float(np.abs(want).max()), 1e-9))
    if err.max() > tol:
        r, c = np.unravel_index(err.argmax(), err.shape)
        first_bad = int(np.argmax(err.max(axis=1) > tol))
        raise AssertionError(f"{what}: max error {err.max():.3e} > {tol:.3e} at row {r}, column {c}; "
                             f"first row over tolerance: {first_bad} of {err.shape[0]}")
