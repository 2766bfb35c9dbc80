"""The layer shapes of the other members of the Qwen3 dense family (the 8B shape has files of its own), two layers
each with a smaller vocabulary, against the plain implementation: widths of 1,024 to 5,120, intermediate sizes of
3,072 to 25,600, 16 to 64 heads over 8 kv heads, tied and untied tables.  Each shape meets tile counts, K ranges and
ring depths of its own in the products, and the 32B shape has more query columns than its width.

The plain implementation runs on the GPU in float64 (the truth) and in the engine's precision (the yardstick), as in
the test of the full-size model: the float32 engine may be at most four times as far from the truth as the plain
float32 implementation, the bfloat16 engine no further than the plain implementation in bfloat16 (a quarter more
is allowed on the maximum of a few hundred thousand values, which moves by that much from draw to draw)."""
import dataclasses
import random
import tempfile

import pytest
import torch

import plain_qwen3 as plain
from qwen_triton_b200 import Engine, StepEntry, load_preset, write_random_model
from qwen_triton_b200.weights import Checkpoint

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
# hidden, intermediate, heads, kv heads, tied tables
SHAPES = {"0.6b": (1024, 3072, 16, 8, True), "1.7b": (2048, 6144, 16, 8, True), "4b": (2560, 9728, 32, 8, True),
          "14b": (5120, 17408, 40, 8, False), "32b": (5120, 25600, 64, 8, False)}
YARDSTICK = {"fp32": (torch.float32, 4.0), "bf16": (torch.bfloat16, 1.25)}


@pytest.fixture(scope="module", params=list(SHAPES))
def member(request):
    hidden, inter, heads, kv, tied = SHAPES[request.param]
    base = load_preset("qwen3-8b")
    config = dataclasses.replace(base, hidden_size=hidden, intermediate_size=inter, num_attention_heads=heads,
                                 num_key_value_heads=kv, num_hidden_layers=2, layer_types=base.layer_types[:2],
                                 vocab_size=20011, tie_word_embeddings=tied, eos_token_id=())
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.set_float32_matmul_precision("highest")
    with tempfile.TemporaryDirectory(prefix="qt_family_") as folder:
        write_random_model(folder, config, seed=11, dtype=torch.bfloat16, device=DEV)
        checkpoint = Checkpoint(folder)
        weights = {name: checkpoint.read(name).to(DEV) for name in checkpoint.names()}
        converted = {dtype: {name: tensor.to(dtype) for name, tensor in weights.items()}
                     for dtype in (torch.float64, torch.float32, torch.bfloat16)}
        yield config, folder, converted
    del weights, converted
    torch.cuda.empty_cache()


def last_logits(cfg, weights, tokens):
    """The plain implementation's logits at the last place of one sequence, in the weights' precision."""
    with torch.no_grad():
        x = plain.embed(torch.tensor(tokens, device=DEV), weights["model.embed_tokens.weight"])
        for index in range(cfg["layers"]):
            x = plain.decoder_layer(x, weights, index, cfg)
        head = weights["model.embed_tokens.weight"] if cfg["tied"] else weights["lm_head.weight"]
        return (plain.rms_norm(x[-1:], weights["model.norm.weight"], cfg["eps"]) @ head.T).double().cpu()


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_a_member_of_the_family(member, dtype):
    config, folder, converted = member
    cfg = plain.read_config(config.to_hf_dict())
    plain_dtype, factor = YARDSTICK[dtype]
    engine = Engine.from_pretrained(folder, dtype=dtype, max_tokens=8192)
    for batch in (1, 8, 33):
        rng = random.Random(batch)
        lengths = [rng.choice([1, 3, 9, 40, 64, 65, 100]) for _ in range(batch)]
        if batch <= 8:
            lengths[0] = 700                                  # a prompt of many token tiles beside the short ones
        generator = torch.Generator().manual_seed(batch)
        prompts = [torch.randint(0, config.vocab_size, (n,), generator=generator).tolist() for n in lengths]
        slots = [engine.new_sequence() for _ in prompts]
        first = engine.step([StepEntry(slot, prompt, [len(prompt) - 1]) for slot, prompt in zip(slots, prompts)])
        stages = [("prompts", first.double().cpu(), [list(prompt) for prompt in prompts])]
        for _ in range(3):
            feed = torch.randint(0, config.vocab_size, (batch,), generator=generator).tolist()
            rows = engine.step([StepEntry(slot, [token], [0]) for slot, token in zip(slots, feed)])
            for prompt, token in zip(prompts, feed):
                prompt.append(token)
        stages.append(("the third one-token step", rows.double().cpu(), prompts))
        for slot in slots:
            engine.release(slot)
        engine.check_kernels()
        for what, got, sequences in stages:
            if batch > 12:                                    # the first and last rows of a large batch
                got, sequences = torch.cat([got[:6], got[-6:]]), sequences[:6] + sequences[-6:]
            truth = torch.cat([last_logits(cfg, converted[torch.float64], s) for s in sequences])
            yard = torch.cat([last_logits(cfg, converted[plain_dtype], s) for s in sequences])
            mine, theirs = (got - truth).abs(), (yard - truth).abs()
            assert float(mine.max()) <= factor * float(theirs.max()), (batch, what, float(mine.max()), float(theirs.max()))
            assert float(mine.pow(2).mean()) <= factor ** 2 * float(theirs.pow(2).mean()), (batch, what)
