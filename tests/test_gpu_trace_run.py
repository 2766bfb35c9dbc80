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
