"""Random weights from a configuration and a seed.

Every tensor is drawn from its own generator keyed by (seed, tensor name), so
the values do not depend on the order of creation or on which other tensors
exist.  Matrices are N(0, initializer_range) as in the reference's
``_reset_parameters`` (qwen_triton/models/core.py:265-272); norm weights are
1 + N(0, 0.1) instead of the reference's constant 1 so that a norm which is
skipped or applied with the wrong weight changes the logits.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Mapping

import torch

from .safetensors_io import write_safetensors
from .tensors import TensorSpec


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 63) - 1)


def random_tensor(name: str, spec: TensorSpec, seed: int, dtype: torch.dtype,
                  device: str | torch.device = "cpu") -> torch.Tensor:
    """Draw one tensor in float32 and round it once to ``dtype``."""
    if spec.role == "table":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    generator = torch.Generator(device=device)
    generator.manual_seed(_tensor_seed(seed, name))
    values = torch.randn(spec.shape, generator=generator, dtype=torch.float32, device=device)
    values = values * spec.init_std + spec.init_mean
    return values.to(dtype)


def random_source(expected: Mapping[str, TensorSpec], seed: int, dtype: torch.dtype,
                  device: str | torch.device = "cpu"):
    """``name -> tensor`` drawing random weights on ``device`` (optional tensors are absent)."""

    def source(name: str):
        spec = expected[name]
        if spec.optional:
            return None
        return random_tensor(name, spec, seed, dtype, device)

    return source


def write_random_model(folder: str | Path, config, seed: int, dtype: torch.dtype = torch.bfloat16) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` with seeded random weights."""
    from ..engine.model import expected_tensors  # parts declare the tensors; no device is touched

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    expected = expected_tensors(config.model_spec())
    tensors = {}
    for name, spec in expected.items():
        if spec.optional:
            continue
        tensors[name] = random_tensor(name, spec, seed, dtype if spec.role != "table" else torch.int32)
    write_safetensors(folder / "model.safetensors", tensors)
    raw = config.to_hf_dict()
    raw["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32"}.get(dtype, str(dtype))
    with (folder / "config.json").open("w", encoding="utf-8") as handle:
        json.dump(raw, handle, indent=2)
    return folder
