"""bin/trace_run driven as a user drives it: JSON steps on standard input, logits files out.  The same
requests are replayed whole, with the last 32 tokens one by one, and in batches of unequal lengths
whose slots are used again, in float32 and bfloat16, and compared with the plain implementation."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from gpu_util import assert_close, model_folder, plain_logits, random_tokens
from qwen_triton_b200 import load_preset

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
PRESET = "tiny-b"
LENGTHS = (40, 7, 65, 1, 33, 90)


def replay(folder, dtype, steps, out_dir, max_tokens):
    lines = "".join(json.dumps(step) + "\n" for step in steps)
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
                           "--out", str(out_dir), "--max-tokens", str(max_tokens)],
                          input=lines, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    done = [line for line in proc.stdout.splitlines() if line.startswith("done ")]
    assert done == [f"done {step['step']}" for step in steps]
    vocab = load_preset(PRESET).vocab_size
    out = {}
    for step in steps:
        path = Path(out_dir) / f"{step['step']}.f32"
        wanted = sum(len(e["want"]) for e in step["entries"])
        if wanted:
            out[step["step"]] = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(wanted, vocab).copy())
        else:
            assert not path.exists()
    return out


@pytest.mark.parametrize("dtype, name", [("float32", "fp32"), ("bfloat16", "bf16")])
def test_trace_replay_three_ways(tmp_path, dtype, name):
    folder = model_folder(PRESET, name)
    requests = {f"r{i}": random_tokens(PRESET, n, 400 + i) for i, n in enumerate(LENGTHS)}

    # 1. each request alone and whole
    steps = [{"step": i, "entries": [{"id": key, "tokens": tokens, "want": list(range(len(tokens)))}], "end": [key]}
             for i, (key, tokens) in enumerate(requests.items())]
    out = replay(folder, dtype, steps, tmp_path / "whole", max_tokens=128)
    for i, (key, tokens) in enumerate(requests.items()):
        assert_close(out[i], plain_logits(PRESET, name, tokens), name, f"whole {key}")

    # 2. the last 32 tokens one by one (a step that wants nothing writes no file)
    steps, owner, number = [], {}, 0
    for key, tokens in requests.items():
        head = max(1, len(tokens) - 32)
        steps.append({"step": number, "entries": [{"id": key, "tokens": tokens[:head], "want": []}], "end": []})
        number += 1
        for at in range(head, len(tokens)):
            steps.append({"step": number, "entries": [{"id": key, "tokens": [tokens[at]], "want": [0]}],
                          "end": [key] if at == len(tokens) - 1 else []})
            owner[number] = (key, at)
            number += 1
        if head == len(tokens):
            steps[-1]["end"] = [key]
    out = replay(folder, dtype, steps, tmp_path / "tail", max_tokens=128)
    for number, (key, at) in owner.items():
        assert_close(out[number], plain_logits(PRESET, name, requests[key])[at:at + 1], name, f"tail32 {key} at {at}")

    # 3. batches of unequal lengths, one after another, in a cache that holds one batch at a time
    steps, owner, number = [], {}, 0
    keys = list(requests)
    for start in range(0, len(keys), 3):
        batch = keys[start:start + 3]
        prompt = {k: max(1, len(requests[k]) // 3) for k in batch}
        entries = [{"id": k, "tokens": requests[k][:prompt[k]], "want": [prompt[k] - 1]} for k in batch]
        steps.append({"step": number, "entries": entries, "end": [k for k in batch if prompt[k] == len(requests[k])]})
        owner[number] = [(k, prompt[k] - 1) for k in batch]
        number += 1
        at = dict(prompt)
        active = [k for k in batch if at[k] < len(requests[k])]
        while active:
            entries = [{"id": k, "tokens": [requests[k][at[k]]], "want": [0]} for k in active]
            owner[number] = [(k, at[k]) for k in active]
            for k in active:
                at[k] += 1
            steps.append({"step": number, "entries": entries, "end": [k for k in active if at[k] == len(requests[k])]})
            number += 1
            active = [k for k in active if at[k] < len(requests[k])]
    out = replay(folder, dtype, steps, tmp_path / "batched", max_tokens=256)
    for number, rows in owner.items():
        expected = torch.stack([plain_logits(PRESET, name, requests[k])[at] for k, at in rows])
        assert_close(out[number], expected, name, f"batched step {number}")


@pytest.mark.parametrize("dtype, name", [("float32", "fp32"), ("bfloat16", "bf16")])
def test_two_batches_live_at_once(tmp_path, dtype, name):
    """A second batch starts while the first still holds its cache, and their one-token steps alternate; requests
    end at different steps, some steps want nothing from a request, and --max-tokens is exactly what the live
    requests hold at the fullest moment (each rounded up to 64)."""
    totals = {"a0": 70, "a1": 33, "a2": 5, "b0": 66, "b1": 2, "b2": 130}
    prompts = {"a0": 60, "a1": 33, "a2": 1, "b0": 3, "b1": 1, "b2": 126}
    requests = {key: random_tokens(PRESET, n, 700 + i) for i, (key, n) in enumerate(totals.items())}
    at, held, steps, owner, peak = {}, {}, [], {}, 0

    def add(entries, own):
        nonlocal peak
        number = len(steps)
        for entry in entries:
            key = entry["id"]
            at[key] = at.get(key, 0) + len(entry["tokens"])
            held[key] = at[key]
        peak = max(peak, sum(-(-n // 64) * 64 for n in held.values()))
        end = [entry["id"] for entry in entries if at[entry["id"]] == totals[entry["id"]]]
        for key in end:
            del held[key]
        steps.append({"step": number, "entries": entries, "end": end})
        if own:
            owner[number] = own

    def start(batch):
        entries = [{"id": k, "tokens": requests[k][:prompts[k]], "want": [0, prompts[k] - 1] if prompts[k] > 1 else [0]} for k in batch]
        add(entries, [(e["id"], w) for e in entries for w in e["want"]])

    def advance(batch, quiet=()):
        active = [k for k in batch if at[k] < totals[k]]
        entries = [{"id": k, "tokens": [requests[k][at[k]]], "want": [] if k in quiet else [0]} for k in active]
        add(entries, [(k, at[k]) for k in active if k not in quiet])
        return bool(active)

    first, second = ["a0", "a1", "a2"], ["b0", "b1", "b2"]
    start(first)
    advance(first)
    start(second)
    turn = 0
    while any(at[k] < totals[k] for k in first + second):
        batch = (first, second)[turn % 2]
        if any(at[k] < totals[k] for k in batch):
            advance(batch, quiet=("a0",) if turn % 3 == 0 else ())
        turn += 1
    assert peak == 64 * 6 and len(steps) == 75            # the schedule itself: six pages at the fullest moment
    out = replay(model_folder(PRESET, name), dtype, steps, tmp_path / "two", max_tokens=peak)
    for number, rows in owner.items():
        expected = torch.stack([plain_logits(PRESET, name, requests[k])[place] for k, place in rows])
        assert_close(out[number], expected, name, f"step {number}: {rows}")
