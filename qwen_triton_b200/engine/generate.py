"""The generation loop above the step function.

Requests (prompts of unequal lengths) are grouped into batches that start together: one step runs
every prompt of the batch, then each further step runs one token per sequence that is still
going.  A sequence ends when it emits a stop token, reaches its token budget or the longest
sequence the cache holds; its slot goes back at once and the others carry on.  Batches follow one
another until every request is served, so slots and pages are used again.

The reference's loop (qwen_triton/models/core.py:392-409) runs a fixed number of greedy steps for a
rectangular batch with no stop condition.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

from ..sampling import SamplingParams
from .step import StepEntry


@dataclass
class GenerationResult:
    tokens: list[int] = field(default_factory=list)
    finish_reason: str = ""      # "stop", "length" or "max_seq_len"


def pages_for(tokens: int, page_tokens: int) -> int:
    return -(-tokens // page_tokens)


def plan_batches(prompt_lengths: Sequence[int], max_new_tokens: int, *, page_tokens: int, total_pages: int,
                 num_slots: int, max_seq_len: int, max_batch_size: int | None = None) -> list[list[int]]:
    """Group request indices, in order, into batches whose sequences all fit the cache at their
    final length (prompt + new tokens, capped by ``max_seq_len``, rounded up to whole pages)."""
    limit = min(num_slots, max_batch_size or num_slots)
    if limit <= 0:
        raise ValueError("a batch needs room for at least one sequence")
    batches: list[list[int]] = []
    current: list[int] = []
    used = 0
    for index, length in enumerate(prompt_lengths):
        if length <= 0:
            raise ValueError(f"request {index} has an empty prompt")
        if length > max_seq_len:
            raise ValueError(f"request {index}: its prompt of {length} tokens exceeds max_seq_len={max_seq_len}")
        need = pages_for(min(length + max_new_tokens, max_seq_len), page_tokens)
        if need > total_pages:
            raise ValueError(f"request {index} needs {need} cache pages, the cache has {total_pages}")
        if current and (len(current) >= limit or used + need > total_pages):
            batches.append(current)
            current, used = [], 0
        current.append(index)
        used += need
    if current:
        batches.append(current)
    return batches


def finish_reason(token: int, produced: int, total_length: int, *, stop_ids: frozenset[int], max_new_tokens: int,
                  max_seq_len: int) -> str:
    """Why a sequence ends after emitting ``token`` as its ``produced``-th new token ('' = it goes on).
    ``total_length`` counts prompt and new tokens, the last one included."""
    if token in stop_ids:
        return "stop"
    if produced >= max_new_tokens:
        return "length"
    if total_length > max_seq_len:       # the new token could not be fed back: the cache holds max_seq_len positions
        return "max_seq_len"
    return ""


def generate(engine, prompts: Sequence[Sequence[int]], *, max_new_tokens: int = 16,
             sampling: SamplingParams | None = None, stop_token_ids: Sequence[int] | None = None,
             ignore_eos: bool = False, max_batch_size: int | None = None, sampler=None) -> list[GenerationResult]:
    """Generate for every prompt; returns one result per prompt, in order.

    ``engine`` offers ``new_sequence()``, ``release(slot)``, ``step(entries) -> logits``,
    ``eos_token_ids``, ``max_seq_len``, ``page_tokens``, ``total_pages`` and ``num_slots``;
    ``sampler.sample(logits, params, requests, steps)`` returns one token id per row.
    """
    sampling = sampling or SamplingParams()
    if sampler is None:
        from ..sampling import Sampler
        sampler = Sampler(engine.device)
    stop_ids = set(stop_token_ids or ())
    if not ignore_eos:
        stop_ids |= set(engine.eos_token_ids)
    stop = frozenset(stop_ids)
    results = [GenerationResult() for _ in prompts]
    if max_new_tokens <= 0:
        for result in results:
            result.finish_reason = "length"
        return results
    batches = plan_batches([len(p) for p in prompts], max_new_tokens, page_tokens=engine.page_tokens,
                           total_pages=engine.total_pages, num_slots=engine.num_slots,
                           max_seq_len=engine.max_seq_len, max_batch_size=max_batch_size)
    for batch in batches:
        slot_of = {index: engine.new_sequence() for index in batch}
        active = list(batch)
        try:
            entries = [StepEntry(slot_of[i], list(prompts[i]), [len(prompts[i]) - 1]) for i in active]
            while active:
                logits = engine.step(entries)
                steps = [len(results[i].tokens) for i in active]
                tokens = sampler.sample(logits, sampling, active, steps)
                still: list[int] = []
                for index, token in zip(active, tokens):
                    result = results[index]
                    result.tokens.append(int(token))
                    reason = finish_reason(int(token), len(result.tokens), len(prompts[index]) + len(result.tokens),
                                           stop_ids=stop, max_new_tokens=max_new_tokens, max_seq_len=engine.max_seq_len)
                    if reason:
                        result.finish_reason = reason
                        engine.release(slot_of.pop(index))
                    else:
                        still.append(index)
                active = still
                entries = [StepEntry(slot_of[i], [results[i].tokens[-1]], [0]) for i in active]
        finally:
            for slot in slot_of.values():
                engine.release(slot)
    return results
