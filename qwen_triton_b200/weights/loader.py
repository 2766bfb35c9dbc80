"""Weights by tensor name, with one clear error for everything that is wrong.

The reference copies what matches and silently skips the rest
(qwen_triton/loaders/hf.py:107-142, report discarded at models/core.py:316).
Here a checkpoint either matches the model's expected tensors exactly or the
load fails with a single message that lists missing tensors, unexpected
tensors and wrong shapes.  Names of wrapped checkpoints are normalised by the
same prefix rules as the reference (loaders/hf.py:80-104).
"""
from __future__ import annotations

from pathlib import Path
from typing import Callable, Mapping

import torch

from .safetensors_io import Checkpoint
from .tensors import TensorSpec

_WRAPPER_PREFIXES = ("model.language_model.model.", "model.language_model.", "language_model.", "model.model.")


class WeightsError(RuntimeError):
    """The checkpoint does not hold exactly the tensors the model needs."""

    def __init__(self, folder, missing, unexpected, wrong_shape):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        lines = [f"checkpoint {folder} does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(self.wrong_shape))
        super().__init__("\n".join(lines))


def _candidates(stored_name: str, expected: Mapping[str, TensorSpec]) -> list[str]:
    out = [stored_name]
    for prefix in _WRAPPER_PREFIXES:
        if stored_name.startswith(prefix):
            stripped = stored_name[len(prefix):]
            out += [stripped, f"model.{stripped}"]
    if stored_name.startswith("model.") and stored_name[6:] in expected:
        out.append(stored_name[6:])
    if not stored_name.startswith("model."):
        out.append(f"model.{stored_name}")
    return out


def match_names(expected: Mapping[str, TensorSpec], stored_names) -> tuple[dict[str, str], list[str]]:
    """Map expected name -> stored name; also return stored names that match nothing."""
    mapping: dict[str, str] = {}
    unexpected: list[str] = []
    for stored in sorted(stored_names):
        for candidate in _candidates(stored, expected):
            if candidate in expected and candidate not in mapping:
                mapping[candidate] = stored
                break
        else:
            unexpected.append(stored)
    return mapping, unexpected


TensorSource = Callable[[str], torch.Tensor]


def open_checkpoint(folder: str | Path, expected: Mapping[str, TensorSpec]) -> TensorSource:
    """Validate the folder against ``expected`` and return ``name -> CPU tensor``.

    Tensors come back in the dtype they are stored in; the parts decide what
    they keep (see :class:`TensorSpec`).
    """
    checkpoint = Checkpoint(folder)
    mapping, unexpected = match_names(expected, checkpoint.tensors)
    missing = [name for name, spec in expected.items() if name not in mapping and not spec.optional]
    wrong = []
    for name, stored_name in mapping.items():
        stored = checkpoint.tensors[stored_name]
        spec = expected[name]
        if tuple(stored.shape) != tuple(spec.shape):
            wrong.append(f"{stored_name}: stored {tuple(stored.shape)}, model needs {tuple(spec.shape)}")
        elif spec.role == "table" and stored.dtype.is_floating_point:
            wrong.append(f"{stored_name}: stored as {stored.dtype}, model needs an integer table")
        elif spec.role != "table" and not stored.dtype.is_floating_point:
            wrong.append(f"{stored_name}: stored as {stored.dtype}, model needs floating point")
    if missing or unexpected or wrong:
        raise WeightsError(folder, sorted(missing), unexpected, wrong)

    def source(name: str) -> torch.Tensor | None:
        if name not in mapping:
            if name in expected and expected[name].optional:
                return None
            raise KeyError(name)
        return checkpoint.read(mapping[name])

    return source


def kept_dtype(spec: TensorSpec, compute_dtype: torch.dtype) -> torch.dtype:
    """Precision a tensor is kept in on the device."""
    if spec.role == "table":
        return torch.int32
    if spec.role == "vector":
        return torch.float32
    return compute_dtype
