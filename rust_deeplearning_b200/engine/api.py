"""The Python entry point, in the manner of the reference's `Generator`
(`rustml/nlp/main/src/core/generator.rs:80-128`: `new`, `with_temperature`, `with_top_k`,
`with_top_p`, `with_repetition_penalty`, `generate`, `generate_stream`, `generate_batch`),
over token ids instead of text: tokenizing is the caller's business.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Union

import torch

from ..config.base import architecture_for, read_config_json
from ..parts.model import Model
from ..sampling.sampler import SamplingParams
from ..weights.loader import load_weights, random_weights
from ..weights.random_init import parse_dtype
from .generate import GenerationResult, GenerationStats, generate
from .step import Engine


def _require_cuda(device):
    dev = torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError("models run on a CUDA device; there is no CPU path")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is available; there is no CPU path")
    return dev


def load_model(folder: str, dtype: Union[str, torch.dtype] = "bfloat16", device="cuda:0", strict: bool = True) -> Model:
    """A model folder (config.json + model.safetensors) -> a model on the device.  The model class
    is chosen by config.json.  dtype "bfloat16": the serving kernels; "float32": everything in
    true 32-bit.  strict False: tensors the model does not read are skipped with a warning instead
    of being an error."""
    dev = _require_cuda(device)
    dtype = parse_dtype(dtype)
    raw = read_config_json(folder)
    arch = architecture_for(raw)
    spec = arch.build_spec(arch.parse_config(raw))
    weights = load_weights(spec, folder, dtype, dev, strict)
    return Model(spec, weights, dtype, dev)


def random_model(config: Dict[str, Any], seed: int = 0, dtype: Union[str, torch.dtype] = "bfloat16",
                 device="cuda:0") -> Model:
    """A model with N(0, 0.02) weights made on the device from (config, seed), without files."""
    dev = _require_cuda(device)
    dtype = parse_dtype(dtype)
    arch = architecture_for(config)
    spec = arch.build_spec(arch.parse_config(config))
    return Model(spec, random_weights(spec, seed, dtype, dev), dtype, dev)


class Generator:
    """Model + cache + sampler.  Options are set with `with_*` calls that return the generator."""

    def __init__(self, model: Model, *, max_cache_tokens: Optional[int] = None, max_batch: int = 64,
                 max_context: Optional[int] = None, use_graphs: bool = True, time_steps: bool = False):
        max_context = min(max_context or model.max_positions, model.max_positions)
        if max_cache_tokens is None:
            max_cache_tokens = max_batch * max_context
        self.model = model
        self.engine = Engine(model, max_tokens=max_cache_tokens, max_seqs=max_batch, max_context=max_context,
                             use_graphs=use_graphs, time_steps=time_steps)
        self._temperature = 0.8
        self._top_k: Optional[int] = None
        self._top_p: Optional[float] = None
        self._repetition_penalty: Optional[float] = None
        self._seed = 0
        self._stop: Optional[frozenset] = None
        self._include_stop = False
        self._bos: Optional[int] = None

    # ---- options (generator.rs:96-128) ----
    def with_temperature(self, temperature: float):
        self._temperature = float(temperature)
        return self

    def with_top_k(self, k: Optional[int]):
        self._top_k = k
        return self

    def with_top_p(self, p: Optional[float]):
        self._top_p = p
        return self

    def with_repetition_penalty(self, penalty: Optional[float]):
        self._repetition_penalty = penalty
        return self

    def with_seed(self, seed: int):
        self._seed = int(seed)
        return self

    def with_eos_token(self, token_id: Optional[int]):
        self._stop = None if token_id is None else frozenset([int(token_id)])
        return self

    def with_stop_tokens(self, token_ids: Optional[Iterable[int]], include_in_output: bool = False):
        self._stop = None if token_ids is None else frozenset(int(t) for t in token_ids)
        self._include_stop = include_in_output
        return self

    def with_bos_token(self, token_id: Optional[int]):
        """Prepend this token to every prompt (generator.rs:245-247)."""
        self._bos = token_id
        return self

    def _params(self) -> SamplingParams:
        return SamplingParams(self._temperature, self._top_k, self._top_p, self._repetition_penalty, self._seed)

    def _prompts(self, prompts):
        out = [list(map(int, p)) for p in prompts]
        if self._bos is not None:
            out = [[int(self._bos)] + p for p in out]
        return out

    # ---- generation ----
    def generate_batch_results(self, prompts: Sequence[Sequence[int]], max_tokens: int = 256,
                               stream: Optional[Callable[[int, int], Optional[bool]]] = None,
                               stats: Optional[GenerationStats] = None) -> List[GenerationResult]:
        return generate(self.engine, self._prompts(prompts), max_new_tokens=max_tokens, sampling=self._params(),
                        stop_token_ids=self._stop, include_stop=self._include_stop, stream=stream, stats=stats)

    def generate(self, prompt: Sequence[int], max_tokens: int = 256) -> List[int]:
        """Prompt plus generated tokens, as the reference returns prompt plus completion (generator.rs:272)."""
        p = self._prompts([prompt])[0]
        return p + self.generate_batch_results([prompt], max_tokens)[0].tokens

    def generate_stream(self, prompt: Sequence[int], max_tokens: int, callback: Callable[[int], Optional[bool]]) -> List[int]:
        """Calls `callback(token)` for every new token; returning False stops (generator.rs:277-318)."""
        p = self._prompts([prompt])[0]
        r = self.generate_batch_results([prompt], max_tokens, stream=lambda _req, tok: callback(tok))
        return p + r[0].tokens

    def generate_batch(self, prompts: Sequence[Sequence[int]], max_tokens: int = 256) -> List[List[int]]:
        """All prompts together in batches of unequal lengths (the reference runs them one by one,
        generator.rs:402-411)."""
        ps = self._prompts(prompts)
        return [p + r.tokens for p, r in zip(ps, self.generate_batch_results(prompts, max_tokens))]
