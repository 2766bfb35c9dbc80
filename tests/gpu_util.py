"""Helpers of the GPU tests: tiny model folders, engines on them, and the plain oracle's logits."""
from __future__ import annotations

import functools
import tempfile
from pathlib import Path

import torch

import plain_qwen3 as plain
from qwen_triton_b200 import Engine, StepEntry, load_preset, write_random_model
from qwen_triton_b200.weights import Checkpoint

# float32: the reference's own bar for model parity (tests/test_model_parity.py:39);
# bfloat16: its bar for bfloat16 kernels (tests/test_kernels.py:150).
TOL = {"fp32": dict(atol=1e-5, rtol=1e-4), "bf16": dict(atol=2e-2, rtol=2e-2)}
STORE = {"fp32": torch.float32, "bf16": torch.bfloat16}
PRESETS = ("tiny-a", "tiny-b", "tiny-c", "tiny-d")      # tiny-d: biased attention projections, head size 64
SEEDS = {"tiny-a": 0, "tiny-b": 1, "tiny-c": 2, "tiny-d": 3}
_KEEP: list = []


@functools.lru_cache(maxsize=None)
def model_folder(preset: str, dtype: str) -> Path:
    """A model folder in a temporary place; weights are stored in the dtype the run computes in, so
    the engine and the oracle see the same values."""
    holder = tempfile.TemporaryDirectory(prefix=f"qt_{preset}_{dtype}_")
    _KEEP.append(holder)
    return write_random_model(holder.name, load_preset(preset), SEEDS[preset], STORE[dtype])


@functools.lru_cache(maxsize=None)
def oracle(preset: str, dtype: str):
    folder = model_folder(preset, dtype)
    checkpoint = Checkpoint(folder)
    weights = {name: checkpoint.read(name).float() for name in checkpoint.names()}
    return load_preset(preset).to_hf_dict(), weights


@functools.lru_cache(maxsize=None)
def _plain_logits(preset: str, dtype: str, tokens: tuple[int, ...]) -> torch.Tensor:
    raw, weights = oracle(preset, dtype)
    return plain.forward(raw, weights, list(tokens))


def plain_logits(preset: str, dtype: str, tokens) -> torch.Tensor:
    return _plain_logits(preset, dtype, tuple(tokens))


def make_engine(preset: str, dtype: str, **kwargs) -> Engine:
    kwargs.setdefault("max_tokens", 2048)
    return Engine.from_pretrained(model_folder(preset, dtype), dtype=dtype, **kwargs)


def random_tokens(preset: str, length: int, seed: int) -> list[int]:
    generator = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, load_preset(preset).vocab_size, (length,), generator=generator).tolist()


def run_whole(engine: Engine, tokens) -> torch.Tensor:
    slot = engine.new_sequence()
    try:
        return engine.step([StepEntry(slot, list(tokens), list(range(len(tokens))))]).cpu()
    finally:
        engine.release(slot)


def assert_close(actual: torch.Tensor, expected: torch.Tensor, dtype: str, what: str = "") -> None:
    actual, expected = actual.float().cpu(), expected.float().cpu()
    assert actual.shape == expected.shape, f"{what}: shape {tuple(actual.shape)} vs {tuple(expected.shape)}"
    tol = TOL[dtype]
    bad = (actual - expected).abs() > tol["atol"] + tol["rtol"] * expected.abs()
    if bad.any():
        rows = bad.reshape(bad.shape[0], -1).any(dim=1).nonzero().flatten().tolist()
        worst = float((actual - expected).abs().max())
        raise AssertionError(f"{what}: {int(bad.sum())} values differ, first wrong row {rows[0]} of {bad.shape[0]} "
                             f"(wrong rows {rows[:12]}), max abs error {worst:.3e}")


@functools.lru_cache(maxsize=None)
def peaky_folder(preset: str, dtype: str, gain: float = 1.5) -> Path:
    """The preset's random model with every q_norm and k_norm weight multiplied by ``gain``: scores spread
    ``gain`` squared times as far, fewer keys carry each softmax, and a key that is missed, misplaced or read
    from the wrong page changes the logits by more (with plain random weights attention over hundreds of keys is
    nearly flat).  The gain also amplifies rounding, smoothly: measured at 1,100 tokens, the worst error over the
    tolerance is 0.03 / 0.16 (float32 / bfloat16) at gain 1, 0.24 / 0.77 at 1.5, 1.06 / 3.2 at 2; 1.5 is the largest
    that leaves the tolerances of the other model tests in place."""
    from qwen_triton_b200.weights import write_safetensors
    source = model_folder(preset, dtype)
    checkpoint = Checkpoint(source)
    tensors = {}
    for name in checkpoint.names():
        tensor = checkpoint.read(name)
        if name.endswith(("q_norm.weight", "k_norm.weight")):
            tensor = (tensor.float() * gain).to(tensor.dtype)
        tensors[name] = tensor
    holder = tempfile.TemporaryDirectory(prefix=f"qt_{preset}_{dtype}_peaky_")
    _KEEP.append(holder)
    folder = Path(holder.name)
    write_safetensors(folder / "model.safetensors", tensors)
    (folder / "config.json").write_text((source / "config.json").read_text())
    return folder


@functools.lru_cache(maxsize=None)
def folder_logits(folder: Path, preset: str, tokens: tuple[int, ...]) -> torch.Tensor:
    """The plain implementation's logits for the model in ``folder``."""
    checkpoint = Checkpoint(folder)
    weights = {name: checkpoint.read(name).float() for name in checkpoint.names()}
    return plain.forward(load_preset(preset).to_hf_dict(), weights, list(tokens))
