"""The generation loop above the step function.

The reference generates one prompt at a time: prefill, sample, then up to max_tokens - 1
times {decode the last token, sample}; a sampled end-of-sequence token ends the sequence and
is neither returned nor fed back; its "batch" API is a sequential map
(`rustml/nlp/main/src/core/generator.rs:243-273, :402-411`).  Here a batch of prompts of
unequal length starts together: all prompts in one step, then one token for each sequence
that is still alive.  Sequences that end earlier leave the batch (their slot is given back);
no request joins a running batch; requests that do not fit run as further batches, one after
another, on the same cache.

`plan_batches` and `SequenceState` hold the loop's decisions and need no device.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Iterable, List, Optional, Sequence

from ..sampling.sampler import Sampler, SamplingParams


@dataclass
class GenerationResult:
    tokens: List[int]          # the new tokens (a stop token is left out unless asked for)
    finish_reason: str         # "stop" | "length" | "context"


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


def generate(engine, prompts: Sequence[Sequence[int]], *, max_new_tokens: int = 256,
             sampling: Optional[SamplingParams] = None, stop_token_ids: Optional[Iterable[int]] = None,
             include_stop: bool = False, stream: Optional[Callable[[int, int], Optional[bool]]] = None,
             max_batch: Optional[int] = None) -> List[GenerationResult]:
    """Generate for every prompt (lists of token ids).

    stop_token_ids: default, the model's end-of-sequence ids.  stream(request index, token) is
    called for every kept token; returning False ends that request (as the reference's streaming
    callback does, generator.rs:277-318)."""
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
            live = list(range(len(seqs)))
            feed = [s.prompt for s in seqs]
            while live:
                logits = engine.step([slots[j] for j in live], feed, "last")
                tokens = sampler.sample(logits, [seqs[j].request for j in live], [seqs[j].sampled for j in live],
                                        [seqs[j].history() for j in live] if need_history else None)
                tokens = tokens.tolist()
                engine.check_status()
                nxt_live, feed = [], []
                for j, tok in zip(live, tokens):
                    s = seqs[j]
                    before = len(s.new_tokens)
                    goes_on = s.accept(int(tok))
                    if stream is not None and len(s.new_tokens) > before:
                        if stream(s.request, int(tok)) is False and goes_on:
                            s.finish_reason, goes_on = "stop", False
                    if goes_on:
                        nxt_live.append(j)
                        feed.append([int(tok)])
                    else:
                        engine.release(slots[j])
                        slots[j] = None
                live = nxt_live
        finally:
            for sl in slots:
                if sl is not None:
                    engine.release(sl)
        for s in seqs:
            results[s.request] = GenerationResult(s.new_tokens, s.finish_reason)
    return results
