"""B200-native generation library for the Qwen3 dense architecture.

Typed configuration and architecture registry, safetensors weights by name, layers assembled from
parts, a paged per-sequence cache, one batched step function, a generation loop, sampling and a
command line, over hand-written CUDA kernels for sm_100a.
"""
from .config import Qwen3Config, config_from_dict, load_config, load_preset, register_architecture
from .engine import Engine, GenerationResult, QwenB200ForCausalLM, StepEntry, generate
from .sampling import SamplingParams
from .weights import WeightsError, write_random_model

__all__ = [
    "Engine", "GenerationResult", "Qwen3Config", "QwenB200ForCausalLM", "SamplingParams", "StepEntry",
    "WeightsError", "config_from_dict", "generate", "load_config", "load_preset", "register_architecture",
    "write_random_model",
]
