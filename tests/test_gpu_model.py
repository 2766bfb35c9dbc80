"""The engine against the plain implementation, in float32 and bfloat16, under every way of cutting
the work: whole, last 32 tokens one by one, unequal batches whose slots are used again, long
decoding, the first tokens, and generation through the entry point."""
import pytest
import torch

import plain_qwen3 as plain
from gpu_util import PRESETS, SEEDS, assert_close, make_engine, model_folder, oracle, plain_logits, random_tokens, run_whole
from qwen_triton_b200 import Engine, QwenB200ForCausalLM, StepEntry, load_preset

pytestmark = pytest.mark.gpu
DTYPES = ("fp32", "bf16")
LENGTHS = {"tiny-a": (5, 9, 17, 70), "tiny-b": (1, 7, 12, 31, 97), "tiny-c": (3, 26, 49, 130), "tiny-d": (2, 21, 66, 140)}


@pytest.fixture(scope="module", params=[(p, d) for p in PRESETS for d in DTYPES], ids=lambda v: f"{v[0]}-{v[1]}")
def case(request):
    preset, dtype = request.param
    # a small chunk limit makes the windowed configuration wrap its ring within the test lengths
    engine = make_engine(preset, dtype, max_tokens=1024, chunk_tokens=16)
    yield preset, dtype, engine
    assert engine.cache.book.live_slots() == []
    engine.cache.book.check()


def requests_of(preset):
    return [random_tokens(preset, n, seed) for seed, n in enumerate(LENGTHS[preset])]


def test_each_request_alone_and_whole(case):
    preset, dtype, engine = case
    for tokens in requests_of(preset):
        assert_close(run_whole(engine, tokens), plain_logits(preset, dtype, tokens), dtype, f"whole, {len(tokens)} tokens")


def test_last_32_tokens_one_by_one(case):
    preset, dtype, engine = case
    for tokens in requests_of(preset):
        if len(tokens) <= 33:
            continue
        head = len(tokens) - 32
        slot = engine.new_sequence()
        rows = [engine.step([StepEntry(slot, tokens[:head], list(range(head)))])]
        for token in tokens[head:]:
            rows.append(engine.step([StepEntry(slot, [token], [0])]))
        engine.release(slot)
        assert_close(torch.cat(rows), plain_logits(preset, dtype, tokens), dtype, f"tail32, {len(tokens)} tokens")


def test_unequal_batches_one_after_another(case):
    """Batches of unequal lengths; prompts in one step, then one token each; shorter requests end
    earlier; the cache is small enough that later batches get the slots and pages of earlier ones."""
    preset, dtype, _ = case
    engine = make_engine(preset, dtype, max_tokens=320, chunk_tokens=16)
    requests = requests_of(preset) + [random_tokens(preset, n, 50 + n) for n in (2, 40, 11, 64, 65)]
    collected = {i: [] for i in range(len(requests))}
    used_slots = []
    for start in range(0, len(requests), 3):
        batch = list(range(start, min(start + 3, len(requests))))
        slots = {i: engine.new_sequence() for i in batch}
        used_slots += list(slots.values())
        prompt = {i: max(1, len(requests[i]) // 2) for i in batch}
        logits = engine.step([StepEntry(slots[i], requests[i][:prompt[i]], list(range(prompt[i]))) for i in batch])
        offset = 0
        for i in batch:
            collected[i].append(logits[offset:offset + prompt[i]])
            offset += prompt[i]
        position = dict(prompt)
        active = [i for i in batch if position[i] < len(requests[i])]
        for i in batch:
            if i not in active:
                engine.release(slots[i])
        while active:
            logits = engine.step([StepEntry(slots[i], [requests[i][position[i]]], [0]) for i in active])
            for row, i in enumerate(active):
                collected[i].append(logits[row:row + 1])
                position[i] += 1
            for i in [i for i in active if position[i] == len(requests[i])]:
                engine.release(slots[i])                       # shorter requests end earlier
            active = [i for i in active if position[i] < len(requests[i])]
        engine.cache.book.check()
    assert len(set(used_slots)) < len(used_slots)              # slots were used again
    for i, tokens in enumerate(requests):
        assert_close(torch.cat(collected[i]), plain_logits(preset, dtype, tokens), dtype, f"batched, request {i} ({len(tokens)} tokens)")


def test_long_decoding(case):
    preset, dtype, engine = case
    tokens = random_tokens(preset, 300, 77)
    slot = engine.new_sequence()
    rows = [engine.step([StepEntry(slot, tokens[:3], [0, 1, 2])])]
    for token in tokens[3:]:
        rows.append(engine.step([StepEntry(slot, [token], [0])]))
    engine.release(slot)
    assert_close(torch.cat(rows), plain_logits(preset, dtype, tokens), dtype, "long decoding")
    assert engine.graph_replays > 200           # the one-token steps ran as replays of a captured step


def test_captured_steps_equal_plain_launches(case):
    """The same decode steps with and without CUDA graphs, at batch sizes that need padding rows."""
    preset, dtype, _ = case
    requests = [random_tokens(preset, n, 600 + n) for n in (70, 3, 41)]
    outputs = []
    for graphs in (True, False):
        engine = make_engine(preset, dtype, max_tokens=1024, chunk_tokens=16, cuda_graphs=graphs)
        slots = [engine.new_sequence() for _ in requests]
        engine.step([StepEntry(s, r[:2], []) for s, r in zip(slots, requests)])
        rows = []
        for at in range(2, 70):
            live = [(s, r) for s, r in zip(slots, requests) if at < len(r)]
            rows.append(engine.step([StepEntry(s, [r[at]], [0]) for s, r in live]))
        outputs.append(torch.cat(rows))
        assert (engine.graph_replays > 0) == graphs
        for s in slots:
            engine.release(s)
    # the same values up to rounding: the captured step runs at a padded shape with its own split counts
    assert_close(outputs[0], outputs[1], dtype, "captured against plain launches")
    expected = torch.cat([torch.stack([plain_logits(preset, dtype, r)[at] for r in requests if at < len(r)]) for at in range(2, 70)])
    assert_close(outputs[0], expected, dtype, "captured steps against the plain implementation")


def test_first_tokens_of_a_sequence(case):
    preset, dtype, engine = case
    tokens = random_tokens(preset, 4, 5)
    slot = engine.new_sequence()
    rows = [engine.step([StepEntry(slot, [t], [0])]) for t in tokens]       # the very first token is a step of its own
    engine.release(slot)
    assert_close(torch.cat(rows), plain_logits(preset, dtype, tokens), dtype, "first tokens")


def test_chunks_of_a_prompt(case):
    """A prompt cut into steps of several tokens (continuation chunks with a past)."""
    preset, dtype, engine = case
    tokens = random_tokens(preset, 75, 9)
    slot = engine.new_sequence()
    rows, start = [], 0
    for size in (7, 1, 30, 20, 17):
        rows.append(engine.step([StepEntry(slot, tokens[start:start + size], list(range(size)))]))
        start += size
    engine.release(slot)
    assert_close(torch.cat(rows), plain_logits(preset, dtype, tokens), dtype, "chunked prompt")


def test_passes_inside_one_step_change_nothing(case):
    """A step larger than the per-pass token limit is cut inside the engine; wanted places keep their order."""
    preset, dtype, _ = case
    engine = make_engine(preset, dtype, max_tokens=1024, max_step_tokens=24, chunk_tokens=16)
    requests = [random_tokens(preset, n, 30 + n) for n in (40, 5, 33)]
    slots = [engine.new_sequence() for _ in requests]
    wants = [[39, 0, 17], [4], list(range(33))]
    logits = engine.step([StepEntry(s, r, w) for s, r, w in zip(slots, requests, wants)])
    for slot in slots:
        engine.release(slot)
    expected = torch.cat([plain_logits(preset, dtype, r)[w] for r, w in zip(requests, wants)])
    assert_close(logits, expected, dtype, "passes inside a step")


def test_greedy_generation_through_the_entry_point(case):
    preset, dtype, _ = case
    raw, weights = oracle(preset, dtype)
    model = QwenB200ForCausalLM.from_pretrained_hf(model_folder(preset, dtype), dtype=dtype, max_tokens=1024)
    prompts = [r[:max(1, len(r) // 2)] for r in requests_of(preset)][:3]
    steps = 8
    results = model.generate(prompts, max_new_tokens=steps, ignore_eos=True)
    for prompt, result in zip(prompts, results):
        assert len(result.tokens) == steps and result.finish_reason == "length"
        if dtype == "fp32":
            assert result.tokens == plain.greedy_generate(raw, weights, prompt, steps)
        else:
            # bfloat16 may pick another token where two logits are closer than its rounding: every chosen
            # token must be within tolerance of the oracle's best at that place, given the engine's own prefix
            sequence = list(prompt)
            for token in result.tokens:
                row = plain.forward(raw, weights, sequence)[-1]
                assert float(row.max() - row[token]) <= 4e-2, (sequence, token)
                sequence.append(token)
    rect = torch.tensor([requests_of(preset)[-1][:6], requests_of(preset)[-1][6:12]])
    out = model.greedy_generate(rect, max_new_tokens=3)
    assert out.shape == (2, 9) and torch.equal(out[:, :6], rect)
    kept = model.forward(rect, logits_to_keep=1).logits
    assert kept.shape == (2, 1, load_preset(preset).vocab_size)
    assert_close(kept[0, 0], plain_logits(preset, dtype, rect[0].tolist())[-1], dtype, "logits_to_keep=1")


def test_temperature_sampling_with_a_fixed_seed():
    """Four prompts of lengths 1/7/12/31, ten steps at temperature 0.8 (float32): the tokens are the
    oracle's inverse-CDF choice with the same uniform numbers (up to float32 rounding of the cumulative weights), and do not depend on the batch."""
    preset, dtype = "tiny-b", "fp32"
    raw, weights = oracle(preset, dtype)
    model = QwenB200ForCausalLM.from_pretrained_hf(model_folder(preset, dtype), dtype=dtype, max_tokens=1024)
    prompts = [random_tokens(preset, n, 200 + n) for n in (1, 7, 12, 31)]
    results = model.generate(prompts, max_new_tokens=10, temperature=0.8, seed=11, ignore_eos=True)
    for index, (prompt, result) in enumerate(zip(prompts, results)):
        sequence = list(prompt)
        for step, token in enumerate(result.tokens):
            row = plain.forward(raw, weights, sequence)[-1]
            assert plain.choice_is_consistent(row, 0.8, plain.uniform_for(11, index, step), token), (index, step)
            sequence.append(token)
    again = model.generate(prompts, max_new_tokens=10, temperature=0.8, seed=11, ignore_eos=True, max_batch_size=2)
    assert [r.tokens for r in again] == [r.tokens for r in results]
    assert [r.tokens for r in model.generate(prompts, max_new_tokens=10, temperature=0.8, seed=12, ignore_eos=True)] != \
        [r.tokens for r in results]


def test_stop_token_ends_a_sequence_early():
    preset, dtype = "tiny-a", "fp32"
    raw, weights = oracle(preset, dtype)
    model = QwenB200ForCausalLM.from_pretrained_hf(model_folder(preset, dtype), dtype=dtype, max_tokens=1024)
    prompts = [random_tokens(preset, n, 300 + n) for n in (5, 9, 17)]
    free_run = [plain.greedy_generate(raw, weights, p, 8) for p in prompts]
    stop = free_run[1][2]
    results = model.generate(prompts, max_new_tokens=8, stop_token_ids=[stop], ignore_eos=True)
    for expected, result in zip(free_run, results):
        cut = expected.index(stop) + 1 if stop in expected else len(expected)
        assert result.tokens == expected[:cut]
        assert result.finish_reason == ("stop" if stop in expected else "length")
    assert model.engine.cache.book.live_slots() == []


def test_a_planned_step_equals_a_plain_one_and_refuses_a_changed_slot(case):
    preset, dtype, engine = case
    prompts = [random_tokens(preset, 7, 910), random_tokens(preset, 3, 911)]
    nexts = [5, 9]
    outs = []
    for planned in (False, True):
        slots = [engine.new_sequence() for _ in prompts]
        engine.step([StepEntry(s, p, []) for s, p in zip(slots, prompts)])
        for _ in range(3):                         # a shape is launched, then captured, then replayed
            if planned:
                plan = engine.plan_decode(slots)
                logits = engine.run_planned(plan, nexts) if plan is not None else engine.step([StepEntry(s, [t], [0]) for s, t in zip(slots, nexts)])
            else:
                logits = engine.step([StepEntry(s, [t], [0]) for s, t in zip(slots, nexts)])
            outs.append(logits.clone())
        if planned and engine.plan_decode(slots[:1]) is not None:
            dropped = engine.plan_decode(slots, extend=True)      # an abandoned plan leaves the extra position behind ...
            again = engine.plan_decode(slots, extend=False)       # ... which a new plan for the same sequences must not take twice
            assert again.lengths == dropped.lengths
            engine.release(slots[1])
            with pytest.raises(ValueError, match="changed since"):
                engine.run_planned(again, nexts)
            engine.release(slots[0])
        else:
            for slot in slots:
                engine.release(slot)
    for a, b in zip(outs[:3], outs[3:]):
        assert_close(b, a, dtype, "planned against plain one-token steps")


def test_errors_are_loud(case):
    preset, dtype, engine = case
    slot = engine.new_sequence()
    with pytest.raises(ValueError, match="outside"):
        engine.step([StepEntry(slot, [load_preset(preset).vocab_size], [0])])
    with pytest.raises(ValueError, match="wanted place"):
        engine.step([StepEntry(slot, [1, 2], [2])])
    with pytest.raises(ValueError, match="twice"):
        engine.step([StepEntry(slot, [1], []), StepEntry(slot, [2], [])])
    engine.release(slot)
    with pytest.raises(ValueError, match="not in use"):
        engine.step([StepEntry(slot, [1], [0])])
    # the refused steps changed nothing: a fresh sequence starts at length 0 and a step of 3 tokens makes it 3
    slot = engine.new_sequence()
    assert engine.length(slot) == 0
    engine.step([StepEntry(slot, [1, 2, 3], [])])
    assert engine.length(slot) == 3
    engine.release(slot)


def test_random_weights_are_the_same_bits_on_the_device_and_on_the_host():
    """``Engine.from_config(seed)`` draws on the device what ``write_random_model(seed)`` writes from the host."""
    from qwen_triton_b200.weights import random_tensor
    from qwen_triton_b200.weights.tensors import TensorSpec
    for name, spec in (("a.weight", TensorSpec((301, 77), init_std=0.02)),
                       ("b.weight", TensorSpec((513,), role="vector", init_std=0.1, init_mean=1.0))):
        for dtype in (torch.float32, torch.bfloat16):
            assert torch.equal(random_tensor(name, spec, 3, dtype, "cuda:0").cpu(), random_tensor(name, spec, 3, dtype))
    preset, dtype = "tiny-b", "bf16"
    tokens = random_tokens(preset, 29, 77)
    drawn = Engine.from_config(load_preset(preset), seed=SEEDS[preset], dtype=dtype, max_tokens=256)
    loaded = make_engine(preset, dtype, max_tokens=256)
    assert torch.equal(run_whole(drawn, tokens), run_whole(loaded, tokens))


@pytest.mark.parametrize("dtype", DTYPES)
def test_biased_projections_with_many_rows_and_with_few(dtype):
    """tiny-d has a bias on q, k, v and o.  A prompt of 300 tokens in one step takes the products for many rows (in
    bfloat16 the block-pair kernel, whose float result the bias is added to), a batch of five one-token steps the
    split products for few; both against the plain implementation."""
    preset = "tiny-d"
    engine = make_engine(preset, dtype, max_tokens=2048)
    long = random_tokens(preset, 300, 900)
    assert_close(run_whole(engine, long), plain_logits(preset, dtype, long), dtype, "300 tokens in one step")
    prompts = [random_tokens(preset, n, 910 + n) for n in (9, 33, 4, 70, 18)]
    slots = [engine.new_sequence() for _ in prompts]
    engine.step([StepEntry(slot, prompt, []) for slot, prompt in zip(slots, prompts)])
    for step in range(3):
        feed = [random_tokens(preset, 1, 950 + 10 * step + i)[0] for i in range(len(prompts))]
        rows = engine.step([StepEntry(slot, [token], [0]) for slot, token in zip(slots, feed)])
        for i, token in enumerate(feed):
            prompts[i].append(token)
            assert_close(rows[i:i + 1], plain_logits(preset, dtype, prompts[i])[-1:], dtype, f"step {step}, request {i}")
    for slot in slots:
        engine.release(slot)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [dict(hidden_size=100, intermediate_size=130, vocab_size=1001, num_attention_heads=5,
                                         num_key_value_heads=1, head_dim=80),
                                    dict(hidden_size=36, intermediate_size=50, vocab_size=77, num_attention_heads=3,
                                         num_key_value_heads=3, head_dim=144),
                                    dict(hidden_size=136, intermediate_size=264, vocab_size=515, num_attention_heads=14,
                                         num_key_value_heads=2, head_dim=16, partial_rotary_factor=0.5)])
def test_sizes_that_fit_no_fast_path(dtype, sizes):
    """Widths that are no multiple of 8 (rows that the tensor-core products and the 16-byte loads do not take), an
    intermediate size that is no multiple of 16 (no interleaved gate and up rows), head sizes beyond 128 and of 16, a
    group of 7 heads, half of a head rotating: the model must pick kernels that take them, in a prompt of two hundred
    tokens and in a batch of one-token steps."""
    import dataclasses, tempfile
    from qwen_triton_b200 import write_random_model
    from qwen_triton_b200.weights import Checkpoint
    base = load_preset("tiny-a")
    config = dataclasses.replace(base, num_hidden_layers=2, layer_types=base.layer_types[:2], tie_word_embeddings=False, **sizes)
    raw = config.to_hf_dict()
    with tempfile.TemporaryDirectory(prefix="qt_odd_") as folder:
        write_random_model(folder, config, seed=12, dtype={"fp32": torch.float32, "bf16": torch.bfloat16}[dtype])
        checkpoint = Checkpoint(folder)
        weights = {name: checkpoint.read(name).float() for name in checkpoint.names()}
        engine = Engine.from_pretrained(folder, dtype=dtype, max_tokens=2048)
    generator = torch.Generator().manual_seed(77)
    prompts = [torch.randint(0, config.vocab_size, (n,), generator=generator).tolist() for n in (200, 3, 61)]
    slots = [engine.new_sequence() for _ in prompts]
    first = engine.step([StepEntry(slot, prompt, list(range(len(prompt)))) for slot, prompt in zip(slots, prompts)])
    expected = torch.cat([plain.forward(raw, weights, prompt) for prompt in prompts])
    assert_close(first, expected, dtype, "prompts")
    for step in range(3):
        feed = torch.randint(0, config.vocab_size, (len(prompts),), generator=generator).tolist()
        rows = engine.step([StepEntry(slot, [token], [0]) for slot, token in zip(slots, feed)])
        for i, token in enumerate(feed):
            prompts[i].append(token)
            assert_close(rows[i:i + 1], plain.forward(raw, weights, prompts[i])[-1:], dtype, f"step {step}, request {i}")
    for slot in slots:
        engine.release(slot)
    engine.check_kernels()
