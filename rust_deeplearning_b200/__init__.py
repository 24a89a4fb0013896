"""A small, whole model library with generation for one GPU (NVIDIA B200, sm_100a).

From a model folder (config.json + safetensors) or a random-weights configuration to
generated tokens: typed configuration and an architecture registry, weights by tensor name,
layers put together from parts, a paged cache with a slot per sequence, one step function,
a generation loop with seeded sampling, and hand-written CUDA kernels underneath.
One architecture is registered: Gemma 2.
"""
from .config import gemma2 as _gemma2  # registers the architecture
from .config.base import ConfigError, load_config, register_architecture, registered_architectures
from .engine.api import Generator, load_model, random_model
from .engine.generate import GenerationResult, generate
from .engine.step import Engine, StepError
from .cache.cache import Cache, CacheError
from .sampling.sampler import SamplingParams
from .weights.loader import WeightError
from .weights.random_init import write_random_model

__all__ = [
    "ConfigError", "load_config", "register_architecture", "registered_architectures",
    "Generator", "load_model", "random_model", "GenerationResult", "generate", "Engine", "StepError",
    "Cache", "CacheError", "SamplingParams", "WeightError", "write_random_model",
]
