"""Dense gated feed-forward: down(act(gate(x)) * up(x)) (qwen_triton/modules/mlp.py:10-22, where act is SiLU;
here it is a parameter: any of ``kernels.ACTIVATIONS``).

gate and up run as one product over the fused weight [gate; up].  In bfloat16 its rows alternate 16 of gate and
16 of up, so that the GEMM for many tokens can apply the SiLU gate in its epilogue (one warp then holds both halves
of 16 features) and write the activation directly; few tokens take the split-K product and the separate kernel,
which reads the same layout.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.kernels import GemmOut
from ..weights.tensors import TensorSpec
from .base import DeferredProduct, Runtime, register_feed_forward
from .linear import Linear


@register_feed_forward("gated_mlp")
class GatedMLP:
    graph_safe = True

    def __init__(self, params, prefix: str, runtime: Runtime) -> None:
        self.prefix = prefix
        self.runtime = runtime
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.activation = params.get("activation", "silu")
        if self.activation not in kernels.ACTIVATIONS:
            raise ValueError(f"{prefix}: gate activation {self.activation!r} is not one of {sorted(kernels.ACTIVATIONS)}")
        self.names = {k: params.get(k, f"{k}_proj") for k in ("gate", "up", "down")}
        fused = runtime.dtype == torch.bfloat16 and self.inter % kernels.SWIGLU_GROUP == 0 and self.hidden % 8 == 0
        self.group = kernels.SWIGLU_GROUP if fused else 0
        self.gate_up = Linear("mlp.gate_up", 2 * self.inter, self.hidden, runtime, role="gate")
        self.down = Linear("mlp.down", self.hidden, self.inter, runtime, role="mlp_out")
        runtime.workspace.declare("mlp.act", runtime.max_step_tokens * self.inter, runtime.dtype)
        # few tokens: the gate in the epilogue of the gate/up product, which then also applies the factor of the norm
        # in front of it (``ScaledRows``)
        self.takes_scaled_rows = bool(self.group) and self.gate_up.fused_capable

    @classmethod
    def expected_tensors(cls, params, prefix: str) -> dict[str, TensorSpec]:
        hidden, inter = int(params["hidden_size"]), int(params["intermediate_size"])
        n = {k: params.get(k, f"{k}_proj") for k in ("gate", "up", "down")}
        return {f"{prefix}.{n['gate']}.weight": TensorSpec((inter, hidden)),
                f"{prefix}.{n['up']}.weight": TensorSpec((inter, hidden)),
                f"{prefix}.{n['down']}.weight": TensorSpec((hidden, inter))}

    def load(self, source) -> None:
        n, p = self.names, self.prefix
        gate, up = source(f"{p}.{n['gate']}.weight"), source(f"{p}.{n['up']}.weight")
        self.gate_up.set_weight(kernels.interleave_gate_up(gate.to(self.runtime.dtype), up.to(self.runtime.dtype), self.group))
        self.down.set_weight(source(f"{p}.{n['down']}.weight"))

    def forward(self, x, ctx):
        tokens = x.shape[0]
        act = self.runtime.workspace.view("mlp.act", tokens, self.inter)
        if self.takes_scaled_rows and self.gate_up.fusable(tokens):
            self.gate_up.into_swiglu(x, act, self.activation)
        elif self.group and kernels.gemm_uses_pairs(x, self.gate_up.weight):
            kernels.gemm_tc_pair(x, self.gate_up.weight, GemmOut(act.view(1, tokens, self.inter)), swiglu=True, activation=self.activation)
        elif self.group and kernels.gemm_tc_supported(x, self.gate_up.weight) and self.gate_up.plan_splits(tokens) == 1:
            # a weight whose tiles fill the machine unsplit: the gate in the plain product's epilogue
            kernels.gemm_tc(x, self.gate_up.weight, GemmOut(act.view(1, tokens, self.inter)), swiglu=True, activation=self.activation)
        else:
            kernels.swiglu(self.gate_up(x), act, self.group, self.activation)
        # few tokens: the down projection is left to the norm behind it, which launches it with the residual addition
        # (and its own preparation) in the product's epilogue
        return DeferredProduct(self.down, act) if self.down.fusable(tokens) else self.down(act)
