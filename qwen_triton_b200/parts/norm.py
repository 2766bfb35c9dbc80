"""RMSNorm fused with the residual addition that precedes it.

y = x * rsqrt(mean(x^2) + eps) * w in float with one rounding at the end, as in the reference
(qwen_triton/kernels/rmsnorm.py:35-42; module qwen_triton/modules/norms.py:9-21).
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.kernels import ScaledRows
from ..weights.tensors import TensorSpec
from .base import ResidualStream, Runtime, register_norm, to_device


@register_norm("rmsnorm")
class RMSNorm:
    graph_safe = True
    offers_scaled_rows = True      # apply(..., lazy=True) may hand on ScaledRows

    def __init__(self, params, name: str, runtime: Runtime) -> None:
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.name = name
        self.runtime = runtime
        self.weight: torch.Tensor | None = None
        runtime.workspace.declare("normed", runtime.max_step_tokens * self.size, runtime.dtype)
        runtime.workspace.declare("normed.sq", -(-self.size // 128) * kernels.FUSED_MAX_ROWS, torch.float32)

    @classmethod
    def expected_tensors(cls, params, name: str) -> dict[str, TensorSpec]:
        return {f"{name}.weight": TensorSpec((int(params["size"]),), role="vector", init_std=0.1, init_mean=1.0)}

    def load(self, source) -> None:
        self.weight = to_device(source(f"{self.name}.weight"), torch.float32, self.runtime.device)

    def apply(self, stream: ResidualStream, rows: torch.Tensor | None = None, lazy: bool = False):
        """Fold the pending delta into the stream and return the normed rows.

        With ``rows`` (int32 row numbers) only those rows are produced and the stream stays as it is.

        Where the pending delta is a product that has not been launched and takes the fused form (few tokens,
        bfloat16), it is launched here with the residual addition in its epilogue.  With ``lazy`` (the consumer is
        a product that takes ``ScaledRows``) the same launch also prepares this norm: it writes the stream times
        the norm's weight and the rows' sums of squares, and the rows' factor is applied by the consumer's
        epilogue; no norm kernel runs.
        """
        ws = self.runtime.workspace
        deferred = stream.take_deferred()
        if deferred is not None:
            count = stream.residual.shape[0]
            if not deferred.linear.fusable(count):
                stream.pending = deferred.run()
            elif rows is None and lazy:
                xw = ws.view("normed", count, self.size)
                sq = ws.view("normed.sq", -(-self.size // 128), count)
                return deferred.linear.into_residual(deferred.x, stream.residual, self.weight, self.eps, xw, sq)
            else:
                deferred.linear.into_residual(deferred.x, stream.residual)
        count = stream.residual.shape[0] if rows is None else rows.shape[0]
        out = ws.view("normed", count, self.size)
        kernels.add_rmsnorm(stream.residual, stream.pending, self.weight, self.eps, out, rows)
        if rows is None:
            stream.pending = None
        return out
