"""The generation loop above the step function.

The reference generates one prompt at a time: prefill, sample, then up to max_tokens - 1
times {decode the last token, sample}; a sampled end-of-sequence token ends the sequence and
is neither returned nor fed back; its "batch" API is a sequential map
(`rustml/nlp/main/src/core/generator.rs:243-273, :402-411`).  Here a batch of prompts of
unequal length starts together: all prompts in one step, then one token for each sequence
that is still alive.  Sequences that end earlier leave the batch (their slot is given back);
no request joins a running batch; requests that do not fit run as further batches, one after
another, on the same cache.

The loop runs one step ahead of what it has read: the step that feeds the sampled tokens back is
queued with the ids still on the device (`Engine.step(..., fed=...)`), and only then are the ids of
the step before read, so the device does not wait for the host between steps.  A sequence whose
last token turns out to be a stop token has then been part of one step too many; that step's token
for it is dropped.  With a repetition penalty the sampler needs every token on the host first, and
the loop waits for each step.

`plan_batches` and `SequenceState` hold the loop's decisions and need no device.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Iterable, List, Optional, Sequence

import torch

from ..sampling.sampler import Sampler, SamplingParams


@dataclass
class GenerationResult:
    tokens: List[int]          # the new tokens (a stop token is left out unless asked for)
    finish_reason: str         # "stop" | "length" | "context"


@dataclass
class GenerationStats:
    """Host wall-clock of a `generate` call, as the reference prints it for its own loop
    (`rustml/nlp/examples/gemma3_gguf.rs:29-75`): the prompts' step up to the first sampled tokens,
    then all single-token steps."""
    prefill_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_tokens: int = 0
    decode_seconds: float = 0.0

    def prefill_rate(self) -> float:
        return self.prefill_tokens / self.prefill_seconds if self.prefill_seconds > 0 else 0.0

    def decode_rate(self) -> float:
        return self.decode_tokens / self.decode_seconds if self.decode_seconds > 0 else 0.0


@dataclass
class SequenceState:
    """One request inside a batch: what it has produced and whether it goes on."""
    request: int                       # index of the request among all requests
    prompt: List[int]
    max_new_tokens: int
    max_context: int
    stop_token_ids: frozenset
    include_stop: bool = False
    new_tokens: List[int] = field(default_factory=list)
    sampled: int = 0                   # tokens sampled so far (keys the random stream)
    finish_reason: Optional[str] = None

    @property
    def finished(self) -> bool:
        return self.finish_reason is not None

    def accept(self, token: int) -> bool:
        """Take the token sampled for this sequence; True if the sequence goes on (the token is
        then fed back).  A stop token ends the sequence and is not kept (generator.rs:253-257,
        :264-268); max_new_tokens counts the first sampled token too (generator.rs:260)."""
        self.sampled += 1
        if token in self.stop_token_ids:
            if self.include_stop:
                self.new_tokens.append(token)
            self.finish_reason = "stop"
            return False
        self.new_tokens.append(token)
        if len(self.new_tokens) >= self.max_new_tokens:
            self.finish_reason = "length"
            return False
        if len(self.prompt) + len(self.new_tokens) > self.max_context:
            # feeding the token back would need one position more than the context has
            self.finish_reason = "context"
            return False
        return True

    def may_go_on_after_one_more(self) -> bool:
        """By the counts alone: could `accept` of one more token, whatever it is, let the sequence go on?"""
        return (not self.finished and len(self.new_tokens) + 1 < self.max_new_tokens
                and len(self.prompt) + len(self.new_tokens) + 1 <= self.max_context)

    def history(self) -> List[int]:
        return self.prompt + self.new_tokens


def plan_batches(prompt_lens: Sequence[int], max_new_tokens: int, *, max_seqs: int, max_tokens: int,
                 page_size: int, max_context: int) -> List[List[int]]:
    """Split requests, in order, into batches that fit the cache: at most `max_seqs` sequences and
    at most `max_tokens` positions, counting every sequence at the longest it can get, rounded up
    to the page size."""
    batches, cur, used = [], [], 0
    for i, n in enumerate(prompt_lens):
        if n < 1:
            raise ValueError(f"request {i}: empty prompt")
        if n > max_context:
            raise ValueError(f"request {i}: prompt of {n} tokens exceeds the context of {max_context}")
        longest = min(n + max(max_new_tokens - 1, 0), max_context)
        cost = -(-longest // page_size) * page_size
        if cost > max_tokens:
            raise ValueError(f"request {i}: needs {cost} cache positions, the cache holds {max_tokens}")
        if cur and (len(cur) >= max_seqs or used + cost > max_tokens):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += cost
    if cur:
        batches.append(cur)
    return batches


class _Readback:
    """Sampled ids on their way to the host: the sampling kernel writes them into pinned memory itself, and
    `tokens()` waits for that kernel alone - not for whatever was queued after it."""

    def __init__(self, sampled, pinned):
        self.sampled, self.n = sampled, sampled.numel()
        self.event = None
        if pinned is not None:
            self.host = pinned[:self.n]
            self.event = torch.cuda.Event()
            self.event.record()

    def tokens(self) -> List[int]:
        if self.event is None:
            return self.sampled.tolist()
        self.event.synchronize()
        return self.host.tolist()


def generate(engine, prompts: Sequence[Sequence[int]], *, max_new_tokens: int = 256,
             sampling: Optional[SamplingParams] = None, stop_token_ids: Optional[Iterable[int]] = None,
             include_stop: bool = False, stream: Optional[Callable[[int, int], Optional[bool]]] = None,
             max_batch: Optional[int] = None, run_ahead: bool = True,
             stats: Optional[GenerationStats] = None) -> List[GenerationResult]:
    """Generate for every prompt (lists of token ids).

    stop_token_ids: default, the model's end-of-sequence ids.  stream(request index, token) is
    called for every kept token; returning False ends that request (as the reference's streaming
    callback does, generator.rs:277-318).  run_ahead False waits for every step's tokens before the
    next step is queued (the results are the same).  stats, if given, receives the call's token counts
    and host times (prompts up to their first sampled tokens; then the single-token steps)."""
    sampling = sampling or SamplingParams()
    model, cache = engine.model, engine.cache
    stops = frozenset(model.spec.stop_token_ids if stop_token_ids is None else stop_token_ids)
    sampler = Sampler(sampling, engine.device)
    prompts = [list(map(int, p)) for p in prompts]
    if max_new_tokens < 1:
        return [GenerationResult([], "length") for _ in prompts]
    max_context = min(cache.max_context, model.max_positions)
    batches = plan_batches([len(p) for p in prompts], max_new_tokens,
                           max_seqs=min(cache.max_seqs, max_batch or cache.max_seqs),
                           max_tokens=cache.max_tokens, page_size=cache.page_size, max_context=max_context)
    results: List[Optional[GenerationResult]] = [None] * len(prompts)
    need_history = sampling.repetition_penalty is not None and not sampling.greedy

    for members in batches:
        seqs = [SequenceState(i, prompts[i], max_new_tokens, max_context, stops, include_stop) for i in members]
        slots = [engine.new_sequence() for _ in seqs]
        try:
            issued = [0] * len(seqs)            # samplings queued per sequence (keys its random stream)
            pinned = None
            if engine.device.type == "cuda":    # two buffers: one being read on the host, one being written by the device
                pinned = [torch.empty(len(seqs), dtype=torch.int32).pin_memory() for _ in range(2)]
            flip = [0]

            def sample(rows, logits):
                flip[0] ^= 1
                host = pinned[flip[0]] if pinned is not None else None
                toks = sampler.sample(logits, [seqs[j].request for j in rows], [issued[j] for j in rows],
                                      [seqs[j].history() for j in rows] if need_history else None, host_out=host)
                for j in rows:
                    issued[j] += 1
                return _Readback(toks, host)

            rows = list(range(len(seqs)))       # the sequences whose tokens `sampled` holds, row by row
            t_start = time.perf_counter()
            sampled = sample(rows, engine.step([slots[j] for j in rows], [s.prompt for s in seqs], "last"))
            ahead = run_ahead and not need_history
            first = True
            while rows:
                nxt_rows, nxt = [], None
                if ahead:
                    # queue the next step before this one's ids are read: everybody who, by the counts, may go on
                    nxt_rows = [j for j in rows if seqs[j].may_go_on_after_one_more()]
                    if nxt_rows:
                        place = {j: i for i, j in enumerate(rows)}
                        logits = engine.step([slots[j] for j in nxt_rows], None, "last",
                                             fed=(sampled.sampled, [place[j] for j in nxt_rows]))
                        nxt = sample(nxt_rows, logits)
                tokens = sampled.tokens()
                engine.check_status()
                if first and stats is not None:
                    # the first tokens are on the host: the prompts' step is over
                    now = time.perf_counter()
                    stats.prefill_tokens += sum(len(s.prompt) for s in seqs)
                    stats.prefill_seconds += now - t_start
                    t_start = now
                first = False
                go_on = []
                for j, tok in zip(rows, tokens):
                    s = seqs[j]
                    if s.finished:
                        continue                # ended a step ago; this token comes from the step queued before that was known
                    before = len(s.new_tokens)
                    goes_on = s.accept(int(tok))
                    if stream is not None and len(s.new_tokens) > before:
                        if stream(s.request, int(tok)) is False and goes_on:
                            s.finish_reason, goes_on = "stop", False
                    if goes_on:
                        go_on.append((j, int(tok)))
                    else:
                        engine.release(slots[j])
                        slots[j] = None
                if ahead:
                    rows, sampled = nxt_rows, nxt
                elif go_on:
                    rows = [j for j, _ in go_on]
                    sampled = sample(rows, engine.step([slots[j] for j in rows], [[tok] for _, tok in go_on], "last"))
                else:
                    rows = []
        finally:
            for sl in slots:
                if sl is not None:
                    engine.release(sl)
        if stats is not None:
            stats.decode_tokens += sum(max(s.sampled - 1, 0) for s in seqs)
            stats.decode_seconds += time.perf_counter() - t_start
        for s in seqs:
            results[s.request] = GenerationResult(s.new_tokens, s.finish_reason)
    return results
