"""Next-token choice: greedy, or temperature sampling with a reproducible random stream.

The reference picks ``argmax`` of the last position and nothing else
(qwen_triton/models/core.py:405).  Temperature sampling here draws token
``softmax(logits / T)`` by inverse CDF in vocabulary order with one uniform number per
(seed, request, step), so a request's tokens do not depend on what else is in the batch.
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

    def __post_init__(self) -> None:
        if self.temperature < 0.0:
            raise ValueError("temperature must not be negative")


def _mix64(value: int) -> int:
    value = (value + 0x9E3779B97F4A7C15) & _MASK64
    value = ((value ^ (value >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    value = ((value ^ (value >> 27)) * 0x94D049BB133111EB) & _MASK64
    return value ^ (value >> 31)


def uniform_for(seed: int, request: int, step: int) -> float:
    """Uniform number in [0, 1) for the ``step``-th new token of request ``request``."""
    state = _mix64(seed & _MASK64)
    state = _mix64(state ^ (request & _MASK64))
    state = _mix64(state ^ (step & _MASK64))
    return (state >> 40) / float(1 << 24)


class Sampler:
    """Chooses one token per logits row on the device and returns the ids to the host."""

    def __init__(self, device: torch.device) -> None:
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, params: SamplingParams, requests: list[int], steps: list[int]) -> list[int]:
        rows = logits.shape[0]
        if rows != len(requests) or rows != len(steps):
            raise ValueError("one request index and one step number per logits row")
        out = torch.empty(rows, dtype=torch.int32, device=self.device)
        if params.temperature == 0.0:
            kernels.argmax(logits, out)
        else:
            uniform = torch.tensor([uniform_for(params.seed, r, s) for r, s in zip(requests, steps)],
                                   dtype=torch.float32).to(self.device)
            temperature = torch.full((rows,), params.temperature, dtype=torch.float32, device=self.device)
            kernels.sample(logits, temperature, uniform, out)
        return out.tolist()
