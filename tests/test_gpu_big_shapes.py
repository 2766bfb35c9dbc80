"""The engine at the layer sizes of the benchmark model (hidden 4096, 32/8 heads of 128, intermediate
12288) with two layers and a smaller vocabulary, against the plain implementation: the tile shapes, split
counts and tensor-core kernels that the tiny configurations never reach.

Sums here run over 4,096 to 12,288 terms and logits reach +-4, so the bars are stated against the float64
result of the plain implementation and scaled to the logits: the float32 engine may be at most four times
as far from it as the plain float32 implementation itself is (both differ from it only by the order of
their float32 sums); the bfloat16 engine at most 2e-2 (the reference's bfloat16 bar,
tests/test_kernels.py:150) of the largest logit."""
import dataclasses
import tempfile

import pytest
import torch

import plain_qwen3 as plain
from qwen_triton_b200 import Engine, StepEntry, load_preset, write_random_model
from qwen_triton_b200.weights import Checkpoint

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def big():
    full = load_preset("qwen3-8b")
    config = dataclasses.replace(full, num_hidden_layers=2, layer_types=full.layer_types[:2], vocab_size=20011,
                                 eos_token_id=())
    with tempfile.TemporaryDirectory(prefix="qt_big_") as folder:
        write_random_model(folder, config, seed=5, dtype=torch.bfloat16)
        checkpoint = Checkpoint(folder)
        weights = {name: checkpoint.read(name).float() for name in checkpoint.names()}
        yield config, folder, weights


def tokens_for(config, length, seed):
    return torch.randint(0, config.vocab_size, (length,), generator=torch.Generator().manual_seed(seed)).tolist()


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_benchmark_layer_shapes_against_the_plain_implementation(big, dtype):
    config, folder, weights = big
    raw = config.to_hf_dict()
    engine = Engine.from_pretrained(folder, dtype=dtype, max_tokens=1024)
    requests = [tokens_for(config, 70, 1), tokens_for(config, 9, 2)]
    truth = [plain.forward(raw, weights, r, dtype=torch.float64) for r in requests]
    plain32 = [plain.forward(raw, weights, r) for r in requests]
    slots = [engine.new_sequence() for _ in requests]
    # prompts of unequal length in one step, then one token each (plain launches, then captured steps)
    prompt = [40, 3]
    got = {0: [], 1: []}
    first = engine.step([StepEntry(s, r[:p], list(range(p))) for s, r, p in zip(slots, requests, prompt)])
    got[0].append(first[:prompt[0]])
    got[1].append(first[prompt[0]:])
    at = list(prompt)
    while any(a < len(r) for a, r in zip(at, requests)):
        live = [i for i in (0, 1) if at[i] < len(requests[i])]
        out = engine.step([StepEntry(slots[i], [requests[i][at[i]]], [0]) for i in live])
        for row, i in enumerate(live):
            got[i].append(out[row:row + 1])
            at[i] += 1
    for slot in slots:
        engine.release(slot)
    for i in (0, 1):
        engine_error = float((torch.cat(got[i]).double().cpu() - truth[i]).abs().max())
        scale = float(truth[i].abs().max())
        if dtype == "fp32":
            plain_error = float((plain32[i].double() - truth[i]).abs().max())
            assert engine_error <= 4 * plain_error + 1e-6, (i, engine_error, plain_error)
        else:
            assert engine_error <= 2e-2 * scale, (i, engine_error, scale)


@pytest.fixture(scope="module")
def mid():
    """Sizes at which the kernels for many tokens and for wide rows take over: hidden 1,024 (a cluster of blocks per
    row in the norms of a decode step), 8/2 heads of 128 (tcgen05 attention, rotation pairs in registers),
    intermediate 2,832 = 16 x 177 (gate and up rows interleaved, the SiLU gate in the GEMM's epilogue)."""
    full = load_preset("qwen3-8b")
    config = dataclasses.replace(full, num_hidden_layers=2, layer_types=full.layer_types[:2], vocab_size=5003, hidden_size=1024,
                                 num_attention_heads=8, num_key_value_heads=2, intermediate_size=2832, eos_token_id=())
    with tempfile.TemporaryDirectory(prefix="qt_mid_") as folder:
        write_random_model(folder, config, seed=6, dtype=torch.bfloat16)
        checkpoint = Checkpoint(folder)
        weights = {name: checkpoint.read(name).float() for name in checkpoint.names()}
        yield config, folder, weights


@pytest.mark.parametrize("prompt", [[300, 290], [150, 97]])
@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_long_prompts_take_the_kernels_for_many_tokens(mid, dtype, prompt):
    """Two prompts of 300 and 290 tokens in one step (more than 256 tokens: block pairs in the products with split K,
    the gated epilogue, the tcgen05 attention), or of 150 and 97 (two token tiles of single blocks, split K), then
    one token each, against the plain implementation in float64."""
    config, folder, weights = mid
    raw = config.to_hf_dict()
    engine = Engine.from_pretrained(folder, dtype=dtype, max_tokens=2048)
    requests = [tokens_for(config, prompt[0] + 6, 3), tokens_for(config, prompt[1] + 3, 4)]
    truth = [plain.forward(raw, weights, r, dtype=torch.float64) for r in requests]
    plain32 = [plain.forward(raw, weights, r) for r in requests]
    slots = [engine.new_sequence() for _ in requests]
    want = [[p for p in (0, 1, 128, 255, 256) if p < prompt[0]] + [prompt[0] - 1], [0, 63, 64, prompt[1] - 1]]
    first = engine.step([StepEntry(s, r[:p], w) for s, r, p, w in zip(slots, requests, prompt, want)])
    got = {0: [first[:len(want[0])]], 1: [first[len(want[0]):]]}
    places = {0: list(want[0]), 1: list(want[1])}
    at = list(prompt)
    while any(a < len(r) for a, r in zip(at, requests)):
        live = [i for i in (0, 1) if at[i] < len(requests[i])]
        out = engine.step([StepEntry(slots[i], [requests[i][at[i]]], [0]) for i in live])
        for row, i in enumerate(live):
            got[i].append(out[row:row + 1])
            places[i].append(at[i])
            at[i] += 1
    for slot in slots:
        engine.release(slot)
    engine.check_kernels()
    for i in (0, 1):
        reference = truth[i][places[i]]
        engine_error = float((torch.cat(got[i]).double().cpu() - reference).abs().max())
        scale = float(reference.abs().max())
        if dtype == "fp32":
            plain_error = float((plain32[i].double()[places[i]] - reference).abs().max())
            assert engine_error <= 4 * plain_error + 1e-6, (i, engine_error, plain_error)
        else:
            assert engine_error <= 2e-2 * scale, (i, engine_error, scale)
