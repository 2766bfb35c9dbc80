"""Configurations drawn at random from everything the architecture's config.json allows, each with a batch of unequal
prompts and some one-token steps, against the plain implementation.  The fixed presets pin the sizes that matter
most; this file walks the space between them: head sizes from 16 to 256 in steps of 16, groups of 1 to 17 heads,
widths from 8 to 2,048 that are or are not multiples of 8, 16 and 128, windows shorter and longer than a page, biased
projections, tied tables, part of a head rotating.  A model is one to three layers; the draw is a function of the
case number alone.

float32 is held to the bar of the other model tests.  bfloat16 is held to the same bar first; where a width of two
thousand puts a few values past it, the engine must be no further from the float64 result than the plain
implementation run in bfloat16 is (the bar of the test of the full-size model)."""
import dataclasses
import random
import tempfile

import pytest
import torch

import plain_qwen3 as plain
from gpu_util import STORE, assert_close
from qwen_triton_b200 import Engine, StepEntry, load_preset, write_random_model
from qwen_triton_b200.weights import Checkpoint

pytestmark = pytest.mark.gpu
CASES = 48


def draw(case: int):
    rng = random.Random(7000 + case)
    kv = rng.choice([1, 1, 2, 3, 4, 5])
    group = rng.choice([1, 1, 2, 3, 4, 6, 7, 8, 12, 16, 17])
    if kv * group > 40:
        group = max(1, 40 // kv)
    layers = rng.choice([1, 2, 3])
    window = rng.choice([None, None, 16, 40, 100, 257])
    kinds = tuple(rng.choice(["full_attention", "sliding_attention"]) if window else "full_attention" for _ in range(layers))
    if window and "sliding_attention" not in kinds:
        kinds = kinds[:-1] + ("sliding_attention",)
    sizes = dict(
        hidden_size=rng.choice([8, 16, 24, 40, 64, 72, 100, 136, 200, 256, 264, 328, 512, 520, 768, 1024, 1032, 2048]),
        intermediate_size=rng.choice([16, 50, 88, 130, 176, 264, 400, 512, 1000, 1536, 1544, 3072]),
        vocab_size=rng.choice([77, 199, 515, 1001, 2048, 5000]),
        num_attention_heads=kv * group, num_key_value_heads=kv,
        head_dim=rng.choice([16, 32, 48, 64, 64, 80, 96, 112, 128, 128, 144, 192, 256]),
        num_hidden_layers=layers, layer_types=kinds, sliding_window=window, use_sliding_window=bool(window),
        max_window_layers=None, tie_word_embeddings=rng.random() < 0.4, attention_bias=rng.random() < 0.3,
        rms_norm_eps=rng.choice([1e-6, 1e-5, 3e-6]), rope_theta=rng.choice([1e4, 2e4, 1e6]),
        partial_rotary_factor=rng.choice([1.0, 1.0, 0.5, 0.25]), max_position_embeddings=4096)
    dtype = ("fp32", "bf16")[case % 2]
    requests = rng.choice([1, 2, 3, 5, 8, 9, 17, 20, 33])
    few = [1, 2, 7, 31, 32, 33, 63, 64, 65, 100, 127, 128, 129, 200, 300, 511, 513, 1100]
    many = [1, 2, 7, 31, 33, 63, 64, 65, 100, 129, 200]
    lengths = [rng.choice(few if requests <= 9 else many) for _ in range(requests)]
    steps = rng.choice([1, 2, 4, 4, 40, 70])
    checked = set(rng.sample(range(steps), min(steps, 3))) | {steps - 1}
    return sizes, dtype, lengths, steps, checked


def compare(rows, prompts, raw, weights, dtype, what):
    expected = torch.cat([plain.forward(raw, weights, prompt)[-1:] for prompt in prompts])
    try:
        assert_close(rows, expected, dtype, what)
    except AssertionError:
        if dtype != "bf16":
            raise
        truth = torch.cat([plain.forward(raw, weights, prompt, dtype=torch.float64)[-1:] for prompt in prompts])
        yard = torch.cat([plain.forward(raw, weights, prompt, dtype=torch.bfloat16)[-1:] for prompt in prompts]).double()
        mine, plain_error = (rows.double().cpu() - truth).abs(), (yard - truth).abs()
        if float(mine.max()) > float(plain_error.max()) or float(mine.pow(2).mean()) > float(plain_error.pow(2).mean()):
            raise


@pytest.mark.parametrize("case, head_dim", [(case, None) for case in range(CASES)] +
                         [(100 + i, d) for i, d in enumerate((2, 6, 10, 24, 40, 50, 72, 100, 250))])
def test_a_random_configuration(case, head_dim):
    """``head_dim`` set: a head size between the steps of 16, which only the kernels for any size take."""
    sizes, dtype, lengths, steps, checked = draw(case)
    if head_dim is not None:
        sizes["head_dim"] = head_dim
    config = dataclasses.replace(load_preset("tiny-a"), **sizes)
    config.validate()
    raw = config.to_hf_dict()
    with tempfile.TemporaryDirectory(prefix="qt_random_") as folder:
        write_random_model(folder, config, seed=case, dtype=STORE[dtype])
        checkpoint = Checkpoint(folder)
        weights = {name: checkpoint.read(name).float() for name in checkpoint.names()}
        engine = Engine.from_pretrained(folder, dtype=dtype, max_tokens=64 * sum((n + steps + 63) // 64 for n in lengths) + 64)
    generator = torch.Generator().manual_seed(case)
    prompts = [torch.randint(0, config.vocab_size, (n,), generator=generator).tolist() for n in lengths]
    slots = [engine.new_sequence() for _ in prompts]
    what = f"{dtype}, lengths {lengths}, " + ", ".join(f"{k}={v}" for k, v in sizes.items())
    first = engine.step([StepEntry(slot, prompt, [len(prompt) - 1]) for slot, prompt in zip(slots, prompts)])
    compare(first, prompts, raw, weights, dtype, f"prompts ({what})")
    for step in range(steps):
        feed = torch.randint(0, config.vocab_size, (len(prompts),), generator=generator).tolist()
        rows = engine.step([StepEntry(slot, [token], [0]) for slot, token in zip(slots, feed)])
        for prompt, token in zip(prompts, feed):
            prompt.append(token)
        if step in checked:
            compare(rows, prompts, raw, weights, dtype, f"step {step} ({what})")
    for slot in slots:
        engine.release(slot)
    engine.check_kernels()


LONG_CASES = 16


def draw_long(case: int):
    """Prompts of thousands of tokens at the head sizes of the tensor-core attention and at others: they arrive whole
    or in steps of 700 or 2,048 tokens, a step takes 1,024 to 4,096 tokens in a pass, and logits are wanted anywhere."""
    rng = random.Random(9000 + case)
    kv, group = rng.choice([1, 2, 3]), rng.choice([1, 2, 4, 5, 8])
    layers = rng.choice([1, 2])
    window = rng.choice([None, None, 100, 257, 1024, 3000])
    kinds = tuple(rng.choice(["full_attention", "sliding_attention"]) if window else "full_attention" for _ in range(layers))
    if window and "sliding_attention" not in kinds:
        kinds = kinds[:-1] + ("sliding_attention",)
    lengths = [rng.choice([1, 65, 1500, 2047, 2048, 2049, 3000, 4097, 6000]) for _ in range(rng.choice([1, 1, 2, 3]))]
    if max(lengths) > 3000 and kv * group > 8:
        group = max(1, 8 // kv)                              # the plain implementation holds every head's whole score matrix
    sizes = dict(
        hidden_size=rng.choice([64, 128, 200, 256, 512]), intermediate_size=rng.choice([88, 256, 512, 1000]),
        vocab_size=rng.choice([199, 1001]), num_attention_heads=kv * group, num_key_value_heads=kv,
        head_dim=rng.choice([64, 64, 128, 128, 128, 32, 96, 256]), num_hidden_layers=layers, layer_types=kinds,
        sliding_window=window, use_sliding_window=bool(window), max_window_layers=None,
        tie_word_embeddings=rng.random() < 0.4, attention_bias=rng.random() < 0.3, rms_norm_eps=1e-6,
        rope_theta=rng.choice([1e4, 1e6]), partial_rotary_factor=rng.choice([1.0, 1.0, 0.5]), max_position_embeddings=8192)
    return sizes, ("bf16", "fp32")[case % 2], lengths, rng.choice([None, None, 700, 2048]), rng.choice([4096, 1024, 2048]), rng.choice([1, 3, 66]), rng


@pytest.mark.parametrize("case", range(LONG_CASES))
def test_a_random_long_prompt(case):
    sizes, dtype, lengths, piece, pass_tokens, steps, rng = draw_long(case)
    config = dataclasses.replace(load_preset("tiny-a"), **sizes)
    config.validate()
    raw = config.to_hf_dict()
    with tempfile.TemporaryDirectory(prefix="qt_random_") as folder:
        write_random_model(folder, config, seed=case, dtype=STORE[dtype])
        checkpoint = Checkpoint(folder)
        weights = {name: checkpoint.read(name).float() for name in checkpoint.names()}
        engine = Engine.from_pretrained(folder, dtype=dtype, max_step_tokens=pass_tokens,
                                        max_tokens=64 * sum((n + steps + 63) // 64 for n in lengths) + 64)
    generator = torch.Generator().manual_seed(case)
    prompts = [torch.randint(0, config.vocab_size, (n,), generator=generator).tolist() for n in lengths]
    whole = [plain.forward(raw, weights, prompt) for prompt in prompts]
    what = f"{dtype}, lengths {lengths} in steps of {piece}, passes of {pass_tokens}, " + ", ".join(f"{k}={v}" for k, v in sizes.items())
    slots = [engine.new_sequence() for _ in prompts]
    fed = [0] * len(prompts)
    piece = piece or max(lengths)
    while any(f < n for f, n in zip(fed, lengths)):
        entries, places = [], []
        for i, (slot, prompt) in enumerate(zip(slots, prompts)):
            part = prompt[fed[i]:fed[i] + piece]
            if part:
                want = sorted(set(rng.sample(range(len(part)), min(len(part), 4))) | {0, len(part) - 1})
                entries.append(StepEntry(slot, part, want))
                places += [(i, fed[i] + w) for w in want]
                fed[i] += len(part)
        rows = engine.step(entries)
        expected = torch.stack([whole[i][place] for i, place in places])
        try:
            assert_close(rows, expected, dtype, f"prompt tokens up to {fed} ({what})")
        except AssertionError:
            compare(rows, [prompts[i][:place + 1] for i, place in places], raw, weights, dtype, what)
    for step in range(steps):
        feed = torch.randint(0, config.vocab_size, (len(prompts),), generator=generator).tolist()
        rows = engine.step([StepEntry(slot, [token], [0]) for slot, token in zip(slots, feed)])
        for prompt, token in zip(prompts, feed):
            prompt.append(token)
        if step in (0, steps - 1):
            compare(rows, prompts, raw, weights, dtype, f"one-token step {step} ({what})")
    for slot in slots:
        engine.release(slot)
    engine.check_kernels()


def test_a_head_size_beyond_the_kernels_is_refused_in_words():
    sizes = draw(0)[0]
    sizes["head_dim"] = 258
    config = dataclasses.replace(load_preset("tiny-a"), **sizes)
    with tempfile.TemporaryDirectory(prefix="qt_random_") as folder:
        write_random_model(folder, config, seed=0, dtype=torch.float32)
        with pytest.raises(ValueError, match="head_dim=258 is beyond what the attention kernels take"):
            Engine.from_pretrained(folder, dtype="fp32", max_tokens=256)
