"""y = x W^T for a weight kept as [out_features, in_features] (qwen_triton/modules/linear.py:11-34).

The weight stays in the layout the checkpoint stores, which is the K-major operand the kernels
read; nothing is transposed per call (the reference re-materialises W^T every call,
qwen_triton/kernels/matmul.py:140).
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.kernels import GemmOut
from .base import Runtime


class Linear:
    def __init__(self, key: str, out_features: int, in_features: int, runtime: Runtime, max_rows: int | None = None,
                 float_out: bool = False) -> None:
        self.key = key
        self.out_features = out_features
        self.in_features = in_features
        self.runtime = runtime
        self.float_out = float_out
        self.weight: torch.Tensor | None = None
        self.max_rows = runtime.max_step_tokens if max_rows is None else max_rows
        self.out_dtype = torch.float32 if float_out else runtime.dtype
        runtime.workspace.declare(f"{key}.out", self.max_rows * out_features, self.out_dtype)

    def set_weight(self, weight: torch.Tensor) -> None:
        if tuple(weight.shape) != (self.out_features, self.in_features):
            raise ValueError(f"{self.key}: weight {tuple(weight.shape)} is not [{self.out_features}, {self.in_features}]")
        self.weight = weight.to(device=self.runtime.device, dtype=self.runtime.dtype).contiguous()

    def __call__(self, x: torch.Tensor, out: torch.Tensor | None = None) -> GemmOut:
        rows = x.shape[0]
        if out is None:
            out = self.runtime.workspace.view(f"{self.key}.out", 1, rows, self.out_features)
        else:
            out = out.view(1, rows, self.out_features)
        result = GemmOut(out)
        kernels.gemm(x, self.weight, result)
        return result
