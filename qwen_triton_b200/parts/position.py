"""Position encodings as tables that the attention kernels read by position.

Rotary: inv_freq[j] = theta^(-2j/rd), angle = pos * inv_freq[j] in float
(qwen_triton/modules/rotary.py:14-26).  The table keeps float cos and sin; the reference rounds
them to the model dtype before use, this library does not.
"""
from __future__ import annotations

import torch

from .base import Runtime, register_position


@register_position("rope")
class RotaryTable:
    def __init__(self, params, runtime: Runtime) -> None:
        self.theta = float(params["theta"])
        self.rotary_dim = int(params["rotary_dim"])
        # which elements turn together: (i, i + rotary_dim / 2) as in the reference (kernels/rope.py:59-69), or
        # neighbours (2i, 2i + 1) with pairing = "interleaved"
        pairing = params.get("pairing", "half")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"rotary pairing {pairing!r} is neither 'half' nor 'interleaved'")
        self.interleaved = pairing == "interleaved"
        if self.rotary_dim % 2 or self.rotary_dim <= 0 or self.rotary_dim > int(params["head_dim"]):
            raise ValueError(f"rotary_dim={self.rotary_dim} must be even and within head_dim={params['head_dim']}")
        self.runtime = runtime

    def key(self) -> tuple:
        return ("rope", self.theta, self.rotary_dim)          # the table does not depend on the pairing

    def table(self, max_positions: int) -> torch.Tensor:
        """float32 [max_positions, rotary_dim]: cos in the first half of each row, sin in the second."""
        exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
        inv_freq = 1.0 / (self.theta ** exponent)
        angles = torch.arange(max_positions, dtype=torch.float32)[:, None] * inv_freq[None, :]
        return torch.cat((angles.cos(), angles.sin()), dim=-1).contiguous().to(self.runtime.device)


@register_position("none")
class NoPosition:
    def __init__(self, params, runtime: Runtime) -> None:
        self.runtime = runtime

    def key(self) -> tuple:
        return ("none",)

    def table(self, max_positions: int):
        return None
