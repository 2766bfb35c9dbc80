"""Next-token choice: greedy, or temperature sampling with a reproducible random stream.

The reference picks ``argmax`` of the last position and nothing else
(qwen_triton/models/core.py:405).  Temperature sampling here draws token
``softmax(logits / T)`` by inverse CDF in vocabulary order with one uniform number per
(seed, request, step), so a request's tokens do not depend on what else is in the batch.
``top_k`` and ``top_p`` (both off by default) leave only the most likely tokens to draw from:
the k largest logits, and of those the smallest set of the most likely whose renormalised
probabilities sum to ``top_p``; tokens that tie with the last one kept are kept as well, so that
the set does not depend on an order among equals.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops import kernels

_MASK64 = (1 << 64) - 1


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0     # 0: greedy (ties go to the lowest token id)
    seed: int = 0
    top_k: int = 0               # > 0: only the k largest logits (with temperature > 0)
    top_p: float = 1.0           # < 1: only the most likely tokens that sum to this share (with temperature > 0)

    def __post_init__(self) -> None:
        if self.temperature < 0.0:
            raise ValueError("temperature must not be negative")
        if self.top_k < 0 or not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_k must not be negative and top_p must lie in (0, 1]")


def _mix64(value: int) -> int:
    value = (value + 0x9E3779B97F4A7C15) & _MASK64
    value = ((value ^ (value >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    value = ((value ^ (value >> 27)) * 0x94D049BB133111EB) & _MASK64
    return value ^ (value >> 31)


def uniform_for(seed: int, request: int, step: int) -> float:
    """Uniform number in [0, 1) for the ``step``-th new token of request ``request``.  The sampling kernel computes
    the same number on the device; this host statement of it is what tests compare with."""
    state = _mix64(seed & _MASK64)
    state = _mix64(state ^ (request & _MASK64))
    state = _mix64(state ^ (step & _MASK64))
    return (state >> 40) / float(1 << 24)


class PendingTokens:
    """Token ids on their way to the host: ``tokens()`` waits for the copy and returns them."""

    def __init__(self, host: torch.Tensor, event: torch.cuda.Event, rows: int, device: torch.Tensor | None = None) -> None:
        self._host, self._event, self._rows = host, event, rows
        self.device = device        # the ids on the device (int32 [rows]), for a step that is queued before the host reads them

    def tokens(self) -> list[int]:
        self._event.synchronize()
        return self._host[:self._rows].tolist()


class Sampler:
    """Chooses one token per logits row on the device and returns the ids to the host."""

    _RING = 4

    def __init__(self, device: torch.device) -> None:
        self.device = torch.device(device)
        self._hosts: list[torch.Tensor] = []     # pinned buffers the ids are copied into, used in turn
        self._keys: list[tuple] = []             # pinned (request, step) buffers, their events and the device copy
        self._turn = 0

    def _keys_on_device(self, requests: list[int], steps: list[int]) -> torch.Tensor:
        """(request, step) per row as int32 [rows, 2] on the device, through a pinned buffer and an asynchronous
        copy: the host does not wait for the device and the device not for the host."""
        rows = len(requests)
        if not self._keys or self._keys[0][0].shape[0] < rows:
            size = max(rows, 64)
            self._keys = [(torch.empty((size, 2), dtype=torch.int32, pin_memory=True), torch.cuda.Event(),
                           torch.empty((size, 2), dtype=torch.int32, device=self.device)) for _ in range(self._RING)]
        host, event, device = self._keys[self._turn % self._RING]
        if self._turn >= self._RING:
            event.synchronize()                  # the copy that last used this buffer has happened
        pairs = host.numpy()
        pairs[:rows, 0] = requests
        pairs[:rows, 1] = steps
        device[:rows].copy_(host[:rows], non_blocking=True)
        event.record()
        return device[:rows]

    def launch(self, logits: torch.Tensor, params: SamplingParams, requests: list[int], steps: list[int]) -> PendingTokens:
        """Start the choice and the copy of the ids to pinned host memory; the caller may do other work before
        it asks the returned object for the tokens."""
        rows = logits.shape[0]
        if rows != len(requests) or rows != len(steps):
            raise ValueError("one request index and one step number per logits row")
        out = torch.empty(rows, dtype=torch.int32, device=self.device)
        if params.temperature == 0.0:
            kernels.argmax(logits, out)
        else:
            kernels.sample_keyed(logits, params.temperature, params.seed, self._keys_on_device(requests, steps), out,
                                 params.top_k, params.top_p)
        if not self._hosts or self._hosts[0].numel() < rows:
            self._hosts = [torch.empty(max(rows, 64), dtype=torch.int32, pin_memory=True) for _ in range(self._RING)]
        host = self._hosts[self._turn % self._RING]
        self._turn += 1
        host[:rows].copy_(out, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return PendingTokens(host, event, rows, out)

    def sample(self, logits: torch.Tensor, params: SamplingParams, requests: list[int], steps: list[int]) -> list[int]:
        return self.launch(logits, params, requests, steps).tokens()
