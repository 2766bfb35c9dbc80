"""Random weights from a configuration and a seed.

Every tensor is drawn from a stream of its own, keyed by (seed, tensor name), so the values do not
depend on the order of creation or on which other tensors exist.  Matrices are N(0, initializer_range)
as in the reference's ``_reset_parameters`` (qwen_triton/models/core.py:265-272); norm weights are
1 + N(0, 0.1) instead of the reference's constant 1 so that a norm which is skipped or applied with the
wrong weight changes the logits.

The draw is the same bits wherever it is made: element ``i`` of a tensor is the sum of twelve 16-bit
fields of three splitmix64 outputs (numbers 3i+1, 3i+2, 3i+3 of the tensor's stream), centred and divided
by 65,536, which is a standard normal to within its twelfth-order Irwin-Hall approximation (tails end at
six sigma).  Only integer operations and two exactly rounded float operations are involved, so a model
drawn on the device (``Engine.from_config``) and a model folder written on the host
(``write_random_model``) hold identical weights for one seed, and an oracle can load the twin of a model
that was never written to disk.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Mapping

import torch

from .safetensors_io import write_safetensors_from
from .tensors import TensorSpec

_MASK64 = (1 << 64) - 1
_GAMMA = 0x9E3779B97F4A7C15          # splitmix64: the stream's increment and the two multipliers of its finaliser
_MUL1 = 0xBF58476D1CE4E5B9
_MUL2 = 0x94D049BB133111EB
_CHUNK = 1 << 24                     # elements drawn at a time (bounds the temporaries)


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 63) - 1)


def _signed(value: int) -> int:
    """The 64-bit pattern ``value`` as the int64 that holds it."""
    value &= _MASK64
    return value - (1 << 64) if value >> 63 else value


def _shift_right(x: torch.Tensor, bits: int) -> torch.Tensor:
    """Logical right shift of int64 (torch's ``>>`` keeps the sign)."""
    return (x >> bits) & ((1 << (64 - bits)) - 1)


def _mix64(x: torch.Tensor) -> torch.Tensor:
    """The splitmix64 finaliser on int64 tensors; products wrap modulo 2^64 on the host and on the device."""
    x = (x ^ _shift_right(x, 30)) * _signed(_MUL1)
    x = (x ^ _shift_right(x, 27)) * _signed(_MUL2)
    return x ^ _shift_right(x, 31)


def standard_normal(stream: int, start: int, count: int, device: str | torch.device = "cpu") -> torch.Tensor:
    """Elements ``start .. start + count`` of the stream ``stream`` as float32 (see the module text)."""
    index = torch.arange(start, start + count, dtype=torch.int64, device=device)
    total = torch.zeros(count, dtype=torch.int64, device=device)
    for j in range(3):
        word = _mix64((index * 3 + (j + 1)) * _signed(_GAMMA) + _signed(stream))
        for field in range(4):
            total += _shift_right(word, 16 * field) & 0xFFFF
    return (total - 393210).to(torch.float32) / 65536.0          # the mean of twelve fields is 12 * 32767.5; all exact in float32


def random_tensor(name: str, spec: TensorSpec, seed: int, dtype: torch.dtype,
                  device: str | torch.device = "cpu", store_dtype: torch.dtype | None = None) -> torch.Tensor:
    """Draw one tensor in float32, round it once to ``store_dtype`` (what a model folder would hold; by default
    ``dtype``) and return it as ``dtype``."""
    if spec.role == "table":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    count = 1
    for dim in spec.shape:
        count *= dim
    out = torch.empty(count, dtype=dtype, device=device)
    stream = _tensor_seed(seed, name)
    for start in range(0, count, _CHUNK):
        size = min(_CHUNK, count - start)
        values = standard_normal(stream, start, size, device) * spec.init_std + spec.init_mean
        out[start:start + size] = values.to(store_dtype or dtype).to(dtype)
    return out.view(spec.shape)


def random_source(expected: Mapping[str, TensorSpec], seed: int, dtype: torch.dtype,
                  device: str | torch.device = "cpu", store_dtype: torch.dtype | None = None):
    """``name -> tensor`` drawing random weights on ``device`` (optional tensors are absent)."""

    def source(name: str):
        spec = expected[name]
        if spec.optional:
            return None
        return random_tensor(name, spec, seed, dtype, device, store_dtype)

    return source


def write_random_model(folder: str | Path, config, seed: int, dtype: torch.dtype = torch.bfloat16,
                       device: str | torch.device = "cpu") -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` with seeded random weights.  ``device`` is
    where the values are drawn (the same bits anywhere; a device draws a large model much faster); they are written
    tensor by tensor."""
    from ..engine.model import expected_tensors  # parts declare the tensors; no device is touched

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    expected = {name: spec for name, spec in expected_tensors(config.model_spec()).items() if not spec.optional}
    entries = {name: (dtype if spec.role != "table" else torch.int32, tuple(spec.shape)) for name, spec in expected.items()}
    write_safetensors_from(folder / "model.safetensors", entries,
                           lambda name: random_tensor(name, expected[name], seed, entries[name][0], device))
    raw = config.to_hf_dict()
    raw["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32"}.get(dtype, str(dtype))
    with (folder / "config.json").open("w", encoding="utf-8") as handle:
        json.dump(raw, handle, indent=2)
    return folder
