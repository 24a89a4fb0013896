"""Sampling parameters and the sampler that turns logits into tokens on the device.

Options and their meaning are the reference's (`rustml/nlp/main/src/core/generator.rs:176-201`,
`rustml/nlp/main/src/core/sampling.rs`): temperature below 1e-7 is greedy arg max (first
maximum wins); otherwise repetition penalty, division by the temperature, top-k, top-p and a
categorical draw, in that order.  The draw is seeded: the uniform number for a row depends
only on (seed, the request's index, how many tokens the request has sampled so far), so a
request's tokens do not depend on what else is in its batch.  The reference draws from an
unseeded thread-local generator (`generator.rs:199`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from ..kernels import ops

GREEDY_BELOW = 1e-7   # generator.rs:177
_M64 = (1 << 64) - 1


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.8                    # the reference's default (infer.rs:27-28); 0 is greedy
    top_k: Optional[int] = None
    top_p: Optional[float] = None
    repetition_penalty: Optional[float] = None
    seed: int = 0

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must not be negative")
        if self.top_k is not None and self.top_k < 1:
            raise ValueError("top_k must be at least 1")
        if self.top_p is not None and not 0 < self.top_p:
            raise ValueError("top_p must be positive")
        if self.repetition_penalty is not None and not self.repetition_penalty > 0:
            raise ValueError("repetition_penalty must be positive")

    @property
    def greedy(self) -> bool:
        return self.temperature < GREEDY_BELOW


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _M64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M64
    return x ^ (x >> 31)


def uniform_for(seed: int, stream: int, step: int) -> float:
    """The uniform number in [0, 1) the sampling kernel uses for (seed, request index, step);
    the same integer hash as in csrc/sampling.cu, 24 bits."""
    h = _splitmix64(seed & _M64)
    h = _splitmix64(h ^ ((stream * 0xD6E8FEB86659FD93) & _M64))
    h = _splitmix64(h ^ ((step * 0xA5A5A5A5A5A5A5A5 + 1) & _M64))
    return float(np.float32(h >> 40) * np.float32(1.0 / 16777216.0))


class Sampler:
    """Samples one token per row of float32 logits on the device."""

    def __init__(self, params: SamplingParams, device):
        self.params = params
        self.device = device

    def sample(self, logits: torch.Tensor, request_ids: Sequence[int], steps: Sequence[int],
               histories: Optional[Sequence[Sequence[int]]] = None, host_out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """logits [rows, vocab]; request_ids and steps key each row's random number; histories (all
        tokens of each row's sequence so far) are needed only with a repetition penalty.
        Returns int32 tokens [rows] on the device; host_out (pinned int32) receives them as well, written by the kernel."""
        p = self.params
        if p.greedy:
            return ops.sample(logits, temperature=0.0, host_out=host_out)
        rows = logits.shape[0]
        stream = torch.tensor(list(request_ids), dtype=torch.int64).to(self.device, non_blocking=True)
        step = torch.tensor(list(steps), dtype=torch.int32).to(self.device, non_blocking=True)
        history = starts = None
        if p.repetition_penalty is not None and p.repetition_penalty != 1.0:
            if histories is None:
                raise ValueError("a repetition penalty needs the sequences' tokens so far")
            offs = np.zeros(rows + 1, dtype=np.int32)
            offs[1:] = np.cumsum([len(h) for h in histories])
            flat = np.concatenate([np.asarray(h, dtype=np.int32) for h in histories]) if offs[-1] else np.zeros(1, np.int32)
            history = torch.from_numpy(flat).to(self.device, non_blocking=True)
            starts = torch.from_numpy(offs).to(self.device, non_blocking=True)
        return ops.sample(logits, temperature=p.temperature, top_k=p.top_k, top_p=p.top_p,
                          repetition_penalty=p.repetition_penalty, seed=p.seed, row_stream=stream, row_step=step,
                          history=history, history_start=starts, host_out=host_out)
