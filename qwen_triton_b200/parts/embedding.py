"""Token embedding into the float residual stream, and the output head.

Embedding: row gather (qwen_triton/modules/embedding.py:9-25).  Head: logits = h W^T without bias,
W being the embedding table itself when tied (qwen_triton/models/core.py:259-263,364); logits are
returned in float.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..weights.tensors import TensorSpec
from .base import Runtime, register_embedding, register_head
from .linear import Linear


@register_embedding("token_embedding")
class TokenEmbedding:
    graph_safe = True

    def __init__(self, params, vocab_size: int, hidden_size: int, runtime: Runtime) -> None:
        self.name = params["name"]
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self.runtime = runtime
        self.table: torch.Tensor | None = None

    @classmethod
    def expected_tensors(cls, params, vocab_size: int, hidden_size: int) -> dict[str, TensorSpec]:
        return {params["name"]: TensorSpec((vocab_size, hidden_size), init_std=float(params.get("init_std", 0.02)))}

    def load(self, source) -> None:
        self.table = source(self.name).to(device=self.runtime.device, dtype=self.runtime.dtype).contiguous()

    def forward(self, token_ids: torch.Tensor, residual: torch.Tensor) -> None:
        kernels.embedding(residual, self.table, token_ids)


@register_head("linear_head")
class LinearHead:
    graph_safe = True

    def __init__(self, params, vocab_size: int, hidden_size: int, runtime: Runtime) -> None:
        self.name = params["name"]
        self.tied_to = params.get("tied_to")
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self.runtime = runtime
        self.linear = Linear("head", vocab_size, hidden_size, runtime, max_rows=0, float_out=True)

    @classmethod
    def expected_tensors(cls, params, vocab_size: int, hidden_size: int) -> dict[str, TensorSpec]:
        # a tied model may still store the head; it is then read past, as in the reference
        return {params["name"]: TensorSpec((vocab_size, hidden_size), optional=params.get("tied_to") is not None)}

    def load(self, source, embedding: TokenEmbedding | None = None) -> None:
        if self.tied_to is not None:
            if embedding is None or embedding.name != self.tied_to:
                raise ValueError(f"head is tied to {self.tied_to!r}, which is not the embedding table")
            self.linear.weight = embedding.table
        else:
            self.linear.set_weight(source(self.name))

    def forward(self, rows: torch.Tensor, out: torch.Tensor) -> None:
        """out [K, vocab] float = rows [K, hidden] W^T."""
        self.linear(rows, out)
