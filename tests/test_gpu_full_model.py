"""The benchmark model itself, all 36 layers of the Qwen3-8B shape with its vocabulary of 151,936, replayed through
``bin/trace_run`` whole, with the last 32 tokens one by one, and in unequal batches whose pages and slots are used
again, in float32 and bfloat16, against the plain implementation (nearest test of the reference:
tests/test_model_parity.py:42-80, one prompt and one cached token at a tiny size).

The plain implementation runs on the GPU here, layer by layer, in float64 (the truth) and, as the yardstick, in the
engine's own precision: float32 with library products in full precision, or bfloat16 rounded where the reference's
bfloat16 model rounds (every product's, norm's and gate's output and the residual sum; float32 inside norms,
rotation, softmax and gate).  Its weights are drawn from the seed that wrote the model folder, rounded to bfloat16
as the folder holds them.  Sums run over 4,096 to 12,288 terms through 36 layers, so the bars are stated against
the truth: the float32 engine may be at most four times as far from it as the plain float32 implementation is (the
bar of the layer-size tests), the bfloat16 engine no further than the plain implementation in bfloat16 (the fixed
2e-2 of the layer-size tests is a bar for two layers; rounding grows with depth)."""
import json
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from qwen_triton_b200 import load_preset, write_random_model
from qwen_triton_b200.engine.model import expected_tensors
from qwen_triton_b200.weights import random_tensor

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
SEED = 21
LENGTHS = {"a": 1100, "b": 300, "c": 70, "d": 33, "e": 640}
EDGES = (0, 63, 64, 255, 256, 511, 512, 1023, 1024)


def checked_places(n: int) -> list[int]:
    """Page and tile edges and the last 32 places."""
    return sorted({p for p in EDGES if p < n} | set(range(max(0, n - 32), n)))


@pytest.fixture(scope="module")
def model():
    config = load_preset("qwen3-8b")
    generator = torch.Generator().manual_seed(SEED)
    requests = {key: torch.randint(0, config.vocab_size, (n,), generator=generator).tolist() for key, n in LENGTHS.items()}
    with tempfile.TemporaryDirectory(prefix="qt_full_") as folder:
        write_random_model(folder, config, seed=SEED, dtype=torch.bfloat16, device="cuda:0")
        yield config, Path(folder), requests


@pytest.fixture(scope="module")
def oracle(model):
    """{float64, float32} -> {request: logits at its checked places}, by the plain implementation's functions."""
    config, _, requests = model
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.set_float32_matmul_precision("highest")
    cfg = plain.read_config(config.to_hf_dict())
    expected = expected_tensors(config.model_spec())

    def draw(name, dtype):
        return random_tensor(name, expected[name], SEED, torch.float32, "cuda:0", store_dtype=torch.bfloat16).to(dtype)

    out = {}
    with torch.no_grad():
        for dtype in (torch.float64, torch.float32, torch.bfloat16):
            table = draw("model.embed_tokens.weight", dtype)
            streams = {key: plain.embed(torch.tensor(tokens, device="cuda:0"), table) for key, tokens in requests.items()}
            del table
            for index in range(cfg["layers"]):
                weights = {name: draw(name, dtype) for name in expected if name.startswith(f"model.layers.{index}.")}
                streams = {key: plain.decoder_layer(x, weights, index, cfg) for key, x in streams.items()}
            norm, head = draw("model.norm.weight", dtype), draw("lm_head.weight", dtype)
            out[dtype] = {key: (plain.rms_norm(x[checked_places(len(x))], norm, cfg["eps"]) @ head.T).cpu()
                          for key, x in streams.items()}
            del streams, weights, norm, head
            torch.cuda.empty_cache()
    return out


def trace(requests):
    """One trace with the three ways of cutting, and for every step that wants logits the (request, place) of each row."""
    steps, rows = [], {}

    def add(entries, end):
        number = len(steps)
        steps.append({"step": number, "entries": [{"id": k, "tokens": t, "want": w} for k, t, w in entries], "end": end})
        return number

    # 1. each request alone and whole
    for key in ("a", "b", "c"):
        places = checked_places(len(requests[key]))
        rows[add([(f"w{key}", requests[key], places)], [f"w{key}"])] = [(key, p) for p in places]
    # 2. the last 32 tokens one by one
    for key in ("a", "c"):
        tokens = requests[key]
        head = len(tokens) - 32
        add([(f"t{key}", tokens[:head], [])], [])
        for at in range(head, len(tokens)):
            rows[add([(f"t{key}", [tokens[at]], [0])], [f"t{key}"] if at == len(tokens) - 1 else [])] = [(key, at)]
    # 3. unequal batches one after another; shorter requests end earlier; the cache holds one batch at a time
    for batch, decoded in ((("a", "b", "c"), {"a": 24, "b": 9, "c": 30}), (("e", "d"), {"e": 12, "d": 20})):
        at = {k: len(requests[k]) - decoded[k] for k in batch}
        number = add([(f"b{k}", requests[k][:at[k]], [at[k] - 1]) for k in batch], [])
        rows[number] = [(k, at[k] - 1) for k in batch]
        active = list(batch)
        while active:
            entries = [(f"b{k}", [requests[k][at[k]]], [0]) for k in active]
            owners = [(k, at[k]) for k in active]
            for k in active:
                at[k] += 1
            done = [k for k in active if at[k] == len(requests[k])]
            rows[add(entries, [f"b{k}" for k in done])] = owners
            active = [k for k in active if k not in done]
    return steps, rows


@pytest.mark.parametrize("dtype, name", [("float32", "fp32"), ("bfloat16", "bf16")])
def test_the_benchmark_model_replayed_three_ways(model, oracle, tmp_path, dtype, name):
    config, folder, requests = model
    steps, rows = trace(requests)
    lines = "".join(json.dumps(step) + "\n" for step in steps)
    # the largest batch holds 1,100 + 300 + 70 tokens, each rounded up to pages of 64: the second batch must reuse them
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
                           "--out", str(tmp_path), "--max-tokens", str(1152 + 320 + 128)],
                          input=lines, capture_output=True, text=True, timeout=1500)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert [line for line in proc.stdout.splitlines() if line.startswith("done ")] == [f"done {s['step']}" for s in steps]
    truth, plain32 = oracle[torch.float64], oracle[torch.float32 if name == "fp32" else torch.bfloat16]
    index_of = {key: {p: i for i, p in enumerate(checked_places(n))} for key, n in LENGTHS.items()}
    worst, yardstick, scale = {}, {}, 0.0
    for number, owners in rows.items():
        got = torch.from_numpy(np.fromfile(tmp_path / f"{number}.f32", dtype="<f4").reshape(len(owners), config.vocab_size).copy())
        for row, (key, place) in enumerate(owners):
            at = index_of[key][place]
            error = float((got[row].double() - truth[key][at]).abs().max())
            label = (steps[number]["entries"][0]["id"][0], key)          # way of cutting (w, t, b) and request
            worst[label] = max(worst.get(label, 0.0), error)
            yardstick[key] = max(yardstick.get(key, 0.0), float((plain32[key][at].double() - truth[key][at]).abs().max()))
            scale = max(scale, float(truth[key][at].abs().max()))
    print(f"{name}: largest logit {scale:.3f}; engine error by (cut, request) {worst}; plain implementation in {name}: {yardstick}")
    for (cut, key), error in worst.items():
        if name == "fp32":
            assert error <= 4 * yardstick[key] + 1e-6, (cut, key, error, yardstick[key])
        else:
            assert error <= yardstick[key], (cut, key, error, yardstick[key])
