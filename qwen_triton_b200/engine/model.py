"""The model as the spec describes it: embedding, blocks run in schedule order, final norm, head.

Counterpart: QwenTritonModel / QwenTritonForCausalLM (qwen_triton/models/core.py:156-263), whose
layer loop (:230-240) runs each layer once in index order; here the order is the spec's
``schedule``.  The final norm and the head run only on the rows whose logits are wanted (the
reference norms every row and then slices, :242,360-364; RMSNorm is row-wise, so the values agree).
"""
from __future__ import annotations

import torch

from ..config.spec import ModelSpec
from ..parts.base import ResidualStream, Runtime, part_class
from ..weights.tensors import TensorSpec


def expected_tensors(spec: ModelSpec) -> dict[str, TensorSpec]:
    """Every checkpoint tensor the model needs, by name.  Touches no device."""
    out: dict[str, TensorSpec] = {}
    out.update(part_class("embedding", spec.embedding).expected_tensors(spec.embedding.params, spec.vocab_size,
                                                                        spec.hidden_size))
    for layer in spec.layers:
        out.update(part_class("block", layer.block).expected_tensors(layer))
    out.update(part_class("norm", spec.final_norm).expected_tensors(spec.final_norm.params, spec.final_norm["name"]))
    out.update(part_class("head", spec.head).expected_tensors(spec.head.params, spec.vocab_size, spec.hidden_size))
    return out


class CausalLM:
    def __init__(self, spec: ModelSpec, runtime: Runtime) -> None:
        spec.validate()
        self.spec = spec
        self.runtime = runtime
        self.embedding = part_class("embedding", spec.embedding)(spec.embedding.params, spec.vocab_size,
                                                                 spec.hidden_size, runtime)
        self.blocks = [part_class("block", layer.block)(layer, runtime) for layer in spec.layers]
        self.final_norm = part_class("norm", spec.final_norm)(spec.final_norm.params, spec.final_norm["name"], runtime)
        self.head = part_class("head", spec.head)(spec.head.params, spec.vocab_size, spec.hidden_size, runtime)
        runtime.workspace.declare("residual", runtime.max_step_tokens * spec.hidden_size, torch.float32)

    def load(self, source) -> None:
        self.embedding.load(source)
        for block in self.blocks:
            block.load(source)
        self.final_norm.load(source)
        self.head.load(source, self.embedding)

    def cache_requests(self) -> list:
        """Per schedule position: what its block keeps per sequence (None for a reader of another position's
        entries): one request, or a list where the block has several parts that keep something."""
        out = []
        for call in self.spec.schedule:
            block = self.blocks[call.layer]
            asked = block.cache_requests() if hasattr(block, "cache_requests") else block.mixer.cache_request()
            out.append(asked if call.cache_of is None else ([None] * len(asked) if isinstance(asked, (list, tuple)) else None))
        return out

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for obj in self._weights():
            if obj.data_ptr() not in seen:
                seen.add(obj.data_ptr())
                total += obj.numel() * obj.element_size()
        return total

    def _weights(self):
        def walk(obj, depth=0):
            if isinstance(obj, torch.Tensor):
                yield obj
            elif depth < 4 and hasattr(obj, "__dict__") and not isinstance(obj, Runtime):
                for key, value in vars(obj).items():
                    if key in ("runtime", "cos_sin"):
                        continue
                    yield from walk(value, depth + 1)
        for part in (self.embedding, *self.blocks, self.final_norm, self.head):
            yield from walk(part)

    def forward(self, ctx, cache, logits: torch.Tensor | None) -> None:
        """Run the tokens of ``ctx`` through every scheduled layer; write the logits of ``ctx.want_rows``."""
        hidden = self.spec.hidden_size
        stream = ResidualStream(self.runtime.workspace.view("residual", ctx.n_tokens, hidden))
        self.embedding.forward(ctx.token_ids, stream.residual)
        for position, call in enumerate(self.spec.schedule):
            self.blocks[call.layer].forward(stream, ctx, cache.view(position))
        if logits is not None and ctx.n_want > 0:
            rows = self.final_norm.apply(stream, rows=ctx.want_rows)
            self.head.forward(rows, logits)
