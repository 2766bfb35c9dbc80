from .api import CausalLMOutput, QwenB200ForCausalLM
from .engine import Engine, parse_dtype
from .generate import BatchRun, GenerationResult, finish_reason, generate, plan_batches
from .model import CausalLM, expected_tensors
from .step import StepContext, StepEntry, plan_passes

__all__ = [
    "BatchRun", "CausalLM", "CausalLMOutput", "Engine", "GenerationResult", "QwenB200ForCausalLM", "StepContext", "StepEntry",
    "expected_tensors", "finish_reason", "generate", "parse_dtype", "plan_batches", "plan_passes",
]
