"""The engine at the schedules that serving and the benchmark run but the small model tests do not reach: one-token
steps with 8, 17 and 64 live rows, more rows than are captured in a CUDA graph, and sequences that are decoded
across position 1,024, where a one-token step's context bucket, page-table width and split counts change.  Every
row is compared with the plain implementation.  The models have their q/k norm weights raised so that a few keys
carry each softmax: a missed or misplaced key then shows in bfloat16 too."""
import dataclasses
import tempfile

import pytest
import torch

import plain_qwen3 as plain
from gpu_util import STORE, assert_close, folder_logits, peaky_folder, random_tokens
from qwen_triton_b200 import Engine, StepEntry, load_preset, write_random_model
from qwen_triton_b200.weights import Checkpoint, write_safetensors

pytestmark = pytest.mark.gpu
DTYPES = ("fp32", "bf16")


def decode_together(engine, requests, prompt_lengths, steps):
    """Prompts of unequal lengths in one step, then ``steps`` one-token steps of all of them; returns per request
    the logits at its prompt's end and at every decoded place."""
    slots = [engine.new_sequence() for _ in requests]
    first = engine.step([StepEntry(s, r[:n], [n - 1]) for s, r, n in zip(slots, requests, prompt_lengths)])
    rows = [[first[i:i + 1]] for i in range(len(requests))]
    for t in range(steps):
        out = engine.step([StepEntry(s, [r[n + t]], [0]) for s, r, n in zip(slots, requests, prompt_lengths)])
        for i in range(len(requests)):
            rows[i].append(out[i:i + 1])
    for slot in slots:
        engine.release(slot)
    engine.check_kernels()
    return [torch.cat(r) for r in rows]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("preset, batch", [("tiny-b", 8), ("tiny-a", 17), ("tiny-b", 64), ("tiny-c", 33)])
def test_one_token_steps_with_many_live_rows(preset, dtype, batch):
    folder = peaky_folder(preset, dtype)
    engine = Engine.from_pretrained(folder, dtype=dtype, max_tokens=batch * 128, chunk_tokens=16)
    steps = 5                                                    # launched, captured, replayed three times
    prompt_lengths = [1 + (7 * i) % 61 for i in range(batch)]
    requests = [random_tokens(preset, n + steps, 2000 + i) for i, n in enumerate(prompt_lengths)]
    got = decode_together(engine, requests, prompt_lengths, steps)
    assert engine.graph_replays >= 3
    for i, (tokens, n) in enumerate(zip(requests, prompt_lengths)):
        assert_close(got[i], folder_logits(folder, preset, tuple(tokens))[n - 1:], dtype, f"row {i} of {batch} (prompt {n})")


@pytest.mark.parametrize("dtype", DTYPES)
def test_more_rows_than_a_captured_step_takes(dtype):
    preset, batch = "tiny-b", 6
    folder = peaky_folder(preset, dtype)
    engine = Engine.from_pretrained(folder, dtype=dtype, max_tokens=1024, max_graph_batch=4)
    prompt_lengths = [3, 40, 1, 17, 64, 9]
    requests = [random_tokens(preset, n + 4, 2100 + i) for i, n in enumerate(prompt_lengths)]
    got = decode_together(engine, requests, prompt_lengths, 4)
    assert engine.graph_replays == 0                             # six rows run as plain launches
    for i, (tokens, n) in enumerate(zip(requests, prompt_lengths)):
        assert_close(got[i], folder_logits(folder, preset, tuple(tokens))[n - 1:], dtype, f"row {i} (prompt {n})")
    # four of them fit a captured step again
    got = decode_together(engine, requests[:4], prompt_lengths[:4], 4)
    assert engine.graph_replays >= 2
    for i, (tokens, n) in enumerate(zip(requests[:4], prompt_lengths[:4])):
        assert_close(got[i], folder_logits(folder, preset, tuple(tokens))[n - 1:], dtype, f"captured row {i} (prompt {n})")


@pytest.mark.parametrize("dtype", DTYPES)
def test_decoding_across_position_1024(dtype):
    """Seven sequences, the longest decoded from 1,000 to 1,100 tokens: the step's context bucket and the page
    table's width change while it runs, for some rows earlier than for others; the configuration has windowed layers
    whose rings wrap many times on the way."""
    preset = "tiny-c"
    folder = peaky_folder(preset, dtype)
    engine = Engine.from_pretrained(folder, dtype=dtype, max_tokens=7 * 1152, max_seq_len=1152, chunk_tokens=32,
                                    max_step_tokens=2048)
    steps = 100
    prompt_lengths = [1000, 990, 1015, 30, 500, 1023, 960]
    requests = [random_tokens(preset, n + steps, 2200 + i) for i, n in enumerate(prompt_lengths)]
    got = decode_together(engine, requests, prompt_lengths, steps)
    buckets = {key[2] for key in engine._graphs}
    assert buckets == {1024, 2048}, buckets
    for i, (tokens, n) in enumerate(zip(requests, prompt_lengths)):
        assert_close(got[i], folder_logits(folder, preset, tuple(tokens))[n - 1:], dtype, f"row {i} (from {n} tokens)")


@pytest.mark.parametrize("dtype", DTYPES)
def test_contexts_of_several_thousand_tokens(dtype):
    """Prompts of 5,000, 4,100 and 70 tokens (the long ones in two passes of a step), then one-token steps: the keys
    of a sequence are cut into 32 ranges, more than a cluster merges, so the partial results go through scratch memory
    and the combine kernel, over page tables of 80 pages.  Raised q/k norm weights let single far keys matter.  The
    plain implementation runs on the device (float32 products, no reduced-precision mode) to keep the test short."""
    base = load_preset("tiny-b")
    config = dataclasses.replace(base, max_position_embeddings=8192)
    raw = config.to_hf_dict()
    with tempfile.TemporaryDirectory(prefix="qt_long_") as folder:
        write_random_model(folder, config, seed=21, dtype=STORE[dtype])
        checkpoint = Checkpoint(folder)
        tensors = {}
        for name in checkpoint.names():
            tensor = checkpoint.read(name)
            if name.endswith(("q_norm.weight", "k_norm.weight")):
                tensor = (tensor.float() * 1.5).to(tensor.dtype)
            tensors[name] = tensor
        write_safetensors(f"{folder}/model.safetensors", tensors)
        engine = Engine.from_pretrained(folder, dtype=dtype, max_tokens=3 * 5120, max_seq_len=5120, max_step_tokens=4096)
    assert not torch.backends.cuda.matmul.allow_tf32
    weights = {name: tensor.float().cuda() for name, tensor in tensors.items()}
    steps = 6
    prompt_lengths = [5000, 4100, 70]
    generator = torch.Generator().manual_seed(31)
    requests = [torch.randint(0, config.vocab_size, (n + steps,), generator=generator).tolist() for n in prompt_lengths]
    got = decode_together(engine, requests, prompt_lengths, steps)
    for i, (tokens, n) in enumerate(zip(requests, prompt_lengths)):
        expected = plain.forward(raw, weights, tokens)[n - 1:].cpu()
        assert_close(got[i], expected, dtype, f"row {i} (from {n} tokens)")
    # alone, a sequence's keys are cut as finely as the scratch allows
    alone = decode_together(engine, requests[:1], prompt_lengths[:1], 3)
    assert_close(alone[0], plain.forward(raw, weights, requests[0])[prompt_lengths[0] - 1:prompt_lengths[0] + 3].cpu(), dtype, "alone")
