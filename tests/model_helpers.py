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


def tolerance(dtype: str, want: np.ndarray) -> float:
    """float32: 5e-5 absolute on logits of order one or less (float32 rounding through a few
    layers).  bfloat16: 3 % of the largest logit (bfloat16 keeps 8 bits; activations are rounded
    a few times per layer) plus a small absolute floor."""
    scale = float(np.abs(want).max())
    return 5e-5 * max(1.0, scale) if dtype == "float32" else 0.03 * scale + 1e-3


def assert_logits(got: torch.Tensor, want: np.ndarray, dtype: str, what=""):
    got = got.detach().float().cpu().double().numpy()
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    err = np.abs(got - want)
    tol = tolerance(dtype, want)
    if err.max() > tol:
        r, c = np.unravel_index(err.argmax(), err.shape)
        first_bad = int(np.argmax(err.max(axis=1) > tol))
        raise AssertionError(f"{what}: max error {err.max():.3e} > {tol:.3e} at row {r}, column {c}; "
                             f"first row over tolerance: {first_bad} of {err.shape[0]}")
