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

import os

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


class BatchRun:
    """One batch of requests that start together: ``start()`` runs every prompt in one step and
    samples each request's first token; every ``advance()`` then feeds the last tokens back, one per
    request that is still going, and samples the next.  Host token ids go in and come out at every step.
    A request that ends gives its slot back at once."""

    def __init__(self, engine, sampler, prompts: Sequence[Sequence[int]], results: list[GenerationResult],
                 indices: Sequence[int], *, max_new_tokens: int, sampling: SamplingParams, stop: frozenset[int]) -> None:
        self.engine, self.sampler = engine, sampler
        self.prompts, self.results = prompts, results
        self.max_new_tokens, self.sampling, self.stop = max_new_tokens, sampling, stop
        self.active = list(indices)
        self.slot_of: dict[int, int] = {}
        self._entries: list[StepEntry] = []
        self._plan = None           # the next one-token step, prepared while the device ran the last one
        self._ahead = None          # (logits, request per row) of a step that is already queued on the device
        self.pipelined = bool(getattr(engine, "accepts_chosen_tokens", False)) and os.environ.get("QT_B200_PIPELINE", "1") != "0"

    @property
    def done(self) -> bool:
        return not self.active

    def start(self) -> list[int]:
        self.slot_of = {index: self.engine.new_sequence() for index in self.active}
        self._entries = [StepEntry(self.slot_of[i], list(self.prompts[i]), [len(self.prompts[i]) - 1]) for i in self.active]
        return self._run()

    def advance(self) -> list[int]:
        return self._run()

    def _ends_whatever_it_emits(self, index: int) -> bool:
        """True if the request's next token is its last by count or by the cache's length, stop token or not."""
        result = self.results[index]
        return bool(finish_reason(-1, len(result.tokens) + 1, len(self.prompts[index]) + len(result.tokens) + 1,
                                  stop_ids=frozenset(), max_new_tokens=self.max_new_tokens,
                                  max_seq_len=self.engine.max_seq_len))

    def _run(self) -> list[int]:
        """One step and one sampled token per active request; returns the tokens in the order of ``active``
        as it was before the step.

        While the device runs the step and the choice of tokens, the host prepares the next one-token step for the
        requests that can only end by a stop token (``plan_decode``, where the engine offers it): that is all of a
        step's host work except putting the tokens in.  Where the engine takes the chosen tokens on the device
        (``accepts_chosen_tokens``) that next step is queued at once, behind the sampling kernel, and only then does
        the host wait for the tokens: the device never waits for the host.  A request that a stop token ends is then
        still a row of the step that is already queued; that row's result is dropped.  Without that, a stop token
        drops the plan, which is made again for those that go on."""
        engine = self.engine
        if self._ahead is not None:                      # queued before the last tokens were read
            logits, order = self._ahead
            self._ahead = None
        else:
            order = list(self.active)
            if self._plan is not None:
                logits = engine.run_planned(self._plan, [self.results[i].tokens[-1] for i in order])
            else:
                logits = engine.step(self._entries)
        self._plan = None
        alive = set(self.active)
        steps = [len(self.results[i].tokens) for i in order]
        launch = getattr(self.sampler, "launch", None)
        planner = getattr(engine, "plan_decode", None)
        plan, expected = None, None
        if launch is not None and planner is not None:
            pending = launch(logits, self.sampling, order, steps)
            expected = [i for i in order if i in alive and not self._ends_whatever_it_emits(i)]
            if expected:
                plan = planner([self.slot_of[i] for i in expected])
            chosen = getattr(pending, "device", None)
            if plan is not None and chosen is not None and self.pipelined:
                row_of = {index: row for row, index in enumerate(order)}
                self._ahead = (engine.run_planned(plan, [row_of[i] for i in expected], chosen=chosen), list(expected))
                plan = None
            tokens = pending.tokens()
        else:
            tokens = self.sampler.sample(logits, self.sampling, order, steps)
        engine.check_kernels(wait=False)                 # the tokens are on the host: their step has finished
        still: list[int] = []
        emitted: list[int] = []
        for index, token in zip(order, tokens):
            if index not in alive:                       # ended by a stop token while this step was already queued
                continue
            emitted.append(int(token))
            result = self.results[index]
            result.tokens.append(int(token))
            reason = finish_reason(int(token), len(result.tokens), len(self.prompts[index]) + len(result.tokens),
                                   stop_ids=self.stop, max_new_tokens=self.max_new_tokens,
                                   max_seq_len=self.engine.max_seq_len)
            if reason:
                result.finish_reason = reason
                self.engine.release(self.slot_of.pop(index))
            else:
                still.append(index)
        self.active = still
        if self._ahead is None:
            if plan is not None and still != expected:   # a stop token: those that go on already have their next position
                plan = planner([self.slot_of[i] for i in still], extend=False) if still else None
            self._plan = plan
            self._entries = [StepEntry(self.slot_of[i], [self.results[i].tokens[-1]], [0]) for i in still]
        return emitted

    def close(self) -> None:
        """Give back whatever the batch still holds (after an error, or when the caller stops early)."""
        for slot in self.slot_of.values():
            self.engine.release(slot)
        self.slot_of = {}
        self.active = []
        self._plan = self._ahead = None


def stop_set(engine, stop_token_ids: Sequence[int] | None, ignore_eos: bool) -> frozenset[int]:
    stop_ids = set(stop_token_ids or ())
    if not ignore_eos:
        stop_ids |= set(engine.eos_token_ids)
    return frozenset(stop_ids)


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
    stop = stop_set(engine, stop_token_ids, ignore_eos)
    results = [GenerationResult() for _ in prompts]
    if max_new_tokens <= 0:
        for result in results:
            result.finish_reason = "length"
        return results
    batches = plan_batches([len(p) for p in prompts], max_new_tokens, page_tokens=engine.page_tokens,
                           total_pages=engine.total_pages, num_slots=engine.num_slots,
                           max_seq_len=engine.max_seq_len, max_batch_size=max_batch_size)
    for batch in batches:
        run = BatchRun(engine, sampler, prompts, results, batch, max_new_tokens=max_new_tokens, sampling=sampling,
                       stop=stop)
        try:
            run.start()
            while not run.done:
                run.advance()
        finally:
            run.close()
    return results
