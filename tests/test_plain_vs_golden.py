"""The plain implementation against logits from the reference's own model code (tests/golden)."""
import importlib.util
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_qwen3 as plain

GOLDEN = Path(__file__).resolve().parent / "golden"
_spec = importlib.util.spec_from_file_location("make_golden", GOLDEN / "make_golden.py")
make_golden = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(make_golden)


@pytest.mark.parametrize("name", sorted(make_golden.CONFIGS))
def test_whole_prompt_logits_match_reference(name):
    raw = make_golden.CONFIGS[name]
    stored = np.load(GOLDEN / f"{name}.npz")
    weights = make_golden.golden_weights(raw, make_golden.SEEDS[name])
    prompt = stored["prompt"].tolist()
    assert prompt == make_golden.golden_prompt(name)
    logits = plain.forward(raw, weights, prompt)
    # the reference's own bar for model parity (tests/test_model_parity.py:39)
    torch.testing.assert_close(logits, torch.from_numpy(stored["logits"]), atol=1e-5, rtol=1e-4)


@pytest.mark.parametrize("name", sorted(make_golden.CONFIGS))
def test_greedy_continuation_matches_reference(name):
    raw = make_golden.CONFIGS[name]
    stored = np.load(GOLDEN / f"{name}.npz")
    weights = make_golden.golden_weights(raw, make_golden.SEEDS[name])
    prompt = stored["prompt"].tolist()[: make_golden.GREEDY_PROMPT]
    assert plain.greedy_generate(raw, weights, prompt, make_golden.GREEDY_NEW) == stored["greedy"].tolist()


def test_window_changes_logits():
    """The windowed golden model must differ from the same weights without a window."""
    raw = dict(make_golden.CONFIGS["golden_c"])
    weights = make_golden.golden_weights(raw, make_golden.SEEDS["golden_c"])
    prompt = make_golden.golden_prompt("golden_c")
    with_window = plain.forward(raw, weights, prompt)
    raw["use_sliding_window"] = False
    without = plain.forward(raw, weights, prompt)
    window = make_golden.CONFIGS["golden_c"]["sliding_window"]
    torch.testing.assert_close(with_window[:window], without[:window], atol=1e-6, rtol=1e-5)
    assert (with_window[window:] - without[window:]).abs().max() > 1e-3


def test_plain_is_causal():
    raw = make_golden.CONFIGS["golden_b"]
    weights = make_golden.golden_weights(raw, 7)
    prompt = make_golden.golden_prompt("golden_b")
    whole = plain.forward(raw, weights, prompt)
    part = plain.forward(raw, weights, prompt[:11])
    torch.testing.assert_close(whole[:11], part, atol=1e-6, rtol=1e-5)


def test_sampling_reference():
    logits = torch.tensor([0.0, 1.0, 2.0, -1.0])
    probs = torch.softmax(logits.double() / 0.8, dim=0)
    edges = torch.cumsum(probs, 0)
    assert plain.sample_temperature(logits, 0.8, 0.0) == 0
    assert plain.sample_temperature(logits, 0.8, float(edges[0]) + 1e-9) == 1
    assert plain.sample_temperature(logits, 0.8, float(edges[1]) + 1e-9) == 2
    assert plain.sample_temperature(logits, 0.8, 0.999999) == 3
    draws = [plain.uniform_for(5, 3, s) for s in range(2000)]
    assert all(0.0 <= u < 1.0 for u in draws) and 0.45 < sum(draws) / len(draws) < 0.55
    assert plain.uniform_for(5, 3, 1) != plain.uniform_for(5, 4, 1) != plain.uniform_for(6, 3, 1)
