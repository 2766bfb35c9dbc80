"""The command line run as a user runs it: ``python -m qwen_triton_b200.scripts.smoke`` as a child process,
its printed tokens compared with the plain implementation (the reference's counterpart is
qwen_triton/scripts/smoke.py:12-72: parse, load, forward, generate, print, optional comparison)."""
import ast
import re
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import plain_qwen3 as plain
from gpu_util import model_folder, oracle, random_tokens
from qwen_triton_b200 import load_preset
from qwen_triton_b200.engine.model import expected_tensors
from qwen_triton_b200.weights import random_tensor

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def run_cli(*options: str) -> str:
    proc = subprocess.run([sys.executable, "-m", "qwen_triton_b200.scripts.smoke", *options], cwd=ROOT,
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    return proc.stdout


def generated(stdout: str) -> list[tuple[list[int], str]]:
    return [(ast.literal_eval(m.group(1)), m.group(2)) for m in re.finditer(r"generated=(\[.*?\]) finish=(\w+)", stdout)]


def ids(tokens) -> str:
    return ",".join(str(t) for t in tokens)


def test_greedy_tokens_of_two_unequal_prompts_equal_the_plain_implementation():
    preset = "tiny-b"
    raw, weights = oracle(preset, "fp32")
    prompts = [random_tokens(preset, 11, 700), random_tokens(preset, 4, 701)]
    out = run_cli("--model-id", str(model_folder(preset, "fp32")), "--dtype", "fp32", "--prompt-ids", ids(prompts[0]),
                  "--prompt-ids", ids(prompts[1]), "--max-new-tokens", "6", "--ignore-eos", "--max-tokens", "512")
    assert "backend=b200" in out
    first = int(plain.forward(raw, weights, prompts[0])[-1].argmax())
    assert f"next_token=[{first}]" in out
    assert generated(out) == [(plain.greedy_generate(raw, weights, p, 6), "length") for p in prompts]


def test_temperature_sampling_and_stop_ids():
    preset = "tiny-a"
    raw, weights = oracle(preset, "fp32")
    prompts = [random_tokens(preset, 9, 710), random_tokens(preset, 5, 711)]
    common = ["--model-id", str(model_folder(preset, "fp32")), "--dtype", "fp32", "--prompt-ids", ids(prompts[0]),
              "--prompt-ids", ids(prompts[1]), "--ignore-eos", "--max-tokens", "512"]
    out = run_cli(*common, "--max-new-tokens", "7", "--temperature", "0.8", "--seed", "11")
    results = generated(out)
    assert [len(tokens) for tokens, _ in results] == [7, 7]
    for index, (prompt, (tokens, _)) in enumerate(zip(prompts, results)):
        sequence = list(prompt)
        for step, token in enumerate(tokens):
            row = plain.forward(raw, weights, sequence)[-1]
            assert plain.choice_is_consistent(row, 0.8, plain.uniform_for(11, index, step), token), (index, step)
            sequence.append(token)
    # drawing from the single most likely token is the greedy choice, whatever the temperature
    results = generated(run_cli(*common, "--max-new-tokens", "6", "--temperature", "0.9", "--top-k", "1"))
    assert results == [(plain.greedy_generate(raw, weights, p, 6), "length") for p in prompts]
    results = generated(run_cli(*common, "--max-new-tokens", "5", "--temperature", "0.9", "--top-p", "0.6", "--seed", "3"))
    for index, (prompt, (tokens, _)) in enumerate(zip(prompts, results)):
        sequence = list(prompt)
        for step, token in enumerate(tokens):
            row = plain.forward(raw, weights, sequence)[-1]
            assert plain.choice_is_consistent(row, 0.9, plain.uniform_for(3, index, step), token, top_p=0.6), (index, step)
            sequence.append(token)
    # a stop token ends its request early and is the last token printed for it
    free_run = [plain.greedy_generate(raw, weights, p, 8) for p in prompts]
    stop = free_run[0][3]
    results = generated(run_cli(*common, "--max-new-tokens", "8", "--stop-ids", str(stop)))
    for expected, (tokens, reason) in zip(free_run, results):
        cut = expected.index(stop) + 1 if stop in expected else len(expected)
        assert tokens == expected[:cut] and reason == ("stop" if stop in expected else "length")


def test_preset_with_random_weights_random_prompts_and_compare_ref():
    """No folder at all: the weights are drawn on the device from --seed.  The same draw on the host gives the
    oracle its model, so the printed tokens can still be checked; --compare-ref sets the bfloat16 run against the
    true 32-bit path on the same (bfloat16-rounded) weights."""
    preset, seed, lengths = "tiny-c", 5, (13, 6, 21)
    config = load_preset(preset)
    out = run_cli("--preset", preset, "--random-weights", "--seed", str(seed), "--dtype", "fp32", "--random-prompts",
                  ids(lengths), "--max-new-tokens", "5", "--ignore-eos", "--max-tokens", "512", "--max-seq-len", "64",
                  "--max-batch-size", "2")
    weights = {name: random_tensor(name, spec, seed, torch.float32) for name, spec in expected_tensors(config.model_spec()).items()
               if not spec.optional}
    generator = torch.Generator().manual_seed(seed)
    prompts = [torch.randint(0, config.vocab_size, (n,), generator=generator).tolist() for n in lengths]
    assert generated(out) == [(plain.greedy_generate(config.to_hf_dict(), weights, p, 5), "length") for p in prompts]

    out = run_cli("--preset", preset, "--random-weights", "--seed", str(seed), "--dtype", "bf16", "--random-prompts", "40",
                  "--max-new-tokens", "2", "--ignore-eos", "--max-tokens", "512", "--compare-ref")
    worst = float(re.search(r"logit_max_abs_diff=([0-9.]+)", out).group(1))
    mean = float(re.search(r"logit_mean_abs_diff=([0-9.]+)", out).group(1))
    assert 0.0 < mean <= worst < 2e-2          # the bar of the bfloat16 model tests (absolute part; logits here are below 1)
