"""Decode and prefill throughput of the Qwen3-8B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl b200|reference] [--temperature T]
    python bench.py --workload 0.6b-unequal | 32b-long

Prints ONE JSON line.  ``value`` is decoded tokens per second at batch 8 from a 2,048-token cache,
timed on the device over the decode steps (step function plus greedy sampling kernel, tokens given
ahead); ``e2e`` is the same through the Python entry point with host token ids in and out at every
step; ``prefill`` is one 2,048-token prompt; ``roofline`` is the decode step's bytes (every weight
once plus the live cache) over its time against the measured HBM copy bandwidth; ``points`` holds
batch 1 and 64 with their fractions.  Weights are random, token ids are uniform random with a fixed seed.

A timed region runs at least K steps and at least ``--min-seconds`` (2 by default): a region of a few
dozen steps is shorter than the clock sampler's period and than the drift of the clocks under the power
cap.  ``steps`` is the number of steps actually timed, ``config.steps_requested`` is K.

``--workload`` runs one of the secondary workloads instead: ``0.6b-unequal`` (Qwen3-0.6B shape, 16 prompts with
lengths uniform in 64..2,048, 128 new tokens each, through ``generate``), ``32b-long`` (Qwen3-32B shape, batch
64 decoded from 2,048 to 4,096 positions, with the roofline fraction in windows of 64 steps near 2,048, 3,072 and 4,096).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def parse_args():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=128)
    parser.add_argument("--warmup", type=int, default=4)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--preset", default="qwen3-8b")
    parser.add_argument("--layers", type=int, default=0, help="run fewer layers than the configuration has (0: all)")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--prompt-len", type=int, default=2048)
    parser.add_argument("--no-points", action="store_true")
    parser.add_argument("--no-prefill", action="store_true")
    parser.add_argument("--min-seconds", type=float, default=2.0, help="a timed region lasts at least this long")
    parser.add_argument("--temperature", type=float, default=0.0, help="sampling temperature of the end-to-end run (0: greedy)")
    parser.add_argument("--workload", default=None, choices=["0.6b-unequal", "32b-long"])
    return parser.parse_args()


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            data = json.loads(path.read_text())
            flat = {}
            for key in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                value = data.get(key)
                if isinstance(value, dict):
                    value = value.get("value")
                if value:
                    flat[key] = float(value)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                return flat, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int = 0) -> None:
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        self.device_index = device_index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-i", str(self.device_index), "-lms", "50"], stdout=self.file,
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        self.file.flush()
        rows = [line.split(",") for line in Path(self.file.name).read_text().splitlines() if line.count(",") >= 5]
        os.unlink(self.file.name)
        clocks, max_clock, reasons = [], 0, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for row in rows:
            try:
                clocks.append(int(row[0]))
                max_clock = max(max_clock, int(row[1]))
            except ValueError:
                continue
            for name, cell in zip(names, row[2:6]):
                if cell.strip().lower() == "active":
                    reasons.add(name)
        return {"sm_mhz": int(statistics.median(clocks)) if clocks else None, "sm_max_mhz": max_clock or None,
                "reasons": sorted(reasons), "samples": len(clocks)}


def random_prompts(batch: int, length: int, vocab: int, seed: int) -> list[list[int]]:
    import torch
    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (batch, length), generator=generator).tolist()


# ----------------------------------------------------------------------------- this library
def model_numbers(config, layers: int) -> dict:
    h, d, nq, nkv, inter, vocab = (config.hidden_size, config.head_dim, config.num_attention_heads,
                                   config.num_key_value_heads, config.intermediate_size, config.vocab_size)
    per_layer = h * (nq + 2 * nkv) * d + nq * d * h + 3 * h * inter
    return {"linear_params": per_layer * layers, "head_params": vocab * h,
            "kv_bytes_per_token": 2 * layers * nkv * d * 2,
            "attn_flops_per_pair": 4 * nq * d * layers}


def steps_for(ms_per_step: float, requested: int, min_seconds: float, most: int) -> int:
    """Steps of a timed region: at least the requested number and at least ``min_seconds`` of them, within ``most``."""
    return max(1, min(most, max(requested, int(min_seconds * 1e3 / max(ms_per_step, 1e-3)) + 1)))


def time_decode(model, prompts, steps: int, warmup: int, vocab: int, min_seconds: float, most_steps: int):
    """Device-timed decode: the batch's cache is filled by a real prefill, then ``warmup`` untimed steps of one
    given token per sequence, each followed by the greedy sampling kernel, then the timed region."""
    import torch
    from qwen_triton_b200 import StepEntry
    from qwen_triton_b200.ops import kernels

    engine = model.engine
    slots = [engine.new_sequence() for _ in prompts]
    for start in range(0, len(prompts), 2):      # fill the cache two prompts at a time
        part = range(start, min(start + 2, len(prompts)))
        engine.step([StepEntry(slots[i], prompts[i], []) for i in part])
    generator = torch.Generator().manual_seed(7)
    out = torch.empty(len(prompts), dtype=torch.int32, device=engine.device)
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def one(tokens):
        logits = engine.step([StepEntry(slot, [tok], [0]) for slot, tok in zip(slots, tokens)])
        kernels.argmax(logits, out)

    probe = 4                                    # untimed steps after the warm-up, only to size the timed region
    feed = torch.randint(0, vocab, (warmup + probe, len(prompts)), generator=generator).tolist()
    for tokens in feed[:warmup]:
        one(tokens)
    torch.cuda.synchronize()
    begin.record()
    for tokens in feed[warmup:]:
        one(tokens)
    end.record()
    torch.cuda.synchronize()
    steps = steps_for(begin.elapsed_time(end) / probe, steps, min_seconds, most_steps)
    warmup += probe
    feed = torch.randint(0, vocab, (steps, len(prompts)), generator=generator).tolist()
    launches = kernels.launch_count()
    with ClockSampler() as clocks:
        begin.record()
        for tokens in feed:
            one(tokens)
        end.record()
        torch.cuda.synchronize()
    launches = kernels.launch_count() - launches
    ms = begin.elapsed_time(end) / steps
    context = len(prompts[0]) + warmup + steps // 2          # mean cache length during the timed steps
    for slot in slots:
        engine.release(slot)
    return ms, launches, clocks.summary(), context, steps


def time_e2e(model, prompts, steps: int, warmup: int, min_seconds: float, most_steps: int, temperature: float = 0.0):
    """Through the entry point: host token ids in, sampled token ids back on the host, every step."""
    import torch
    run = model.start_batch(prompts, max_new_tokens=warmup + most_steps + 8, temperature=temperature, seed=5, ignore_eos=True)
    run.start()
    for _ in range(warmup):
        run.advance()
    torch.cuda.synchronize()
    wall = time.perf_counter()
    for _ in range(4):                           # untimed, only to size the timed region
        run.advance()
    torch.cuda.synchronize()
    steps = steps_for((time.perf_counter() - wall) * 1e3 / 4, steps, min_seconds, most_steps)
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall = time.perf_counter()
    begin.record()
    for _ in range(steps):
        run.advance()
    end.record()
    torch.cuda.synchronize()
    wall = (time.perf_counter() - wall) * 1e3 / steps
    ms = max(begin.elapsed_time(end) / steps, wall)
    h2d = model.engine.last_meta_bytes + (8 * len(prompts) if temperature > 0 else 0)     # sampling keys: request and step per row
    run.close()
    return ms, h2d, 4 * len(prompts), steps


def time_prefill(model, tokens: int, vocab: int, repeats: int = 5, warmup: int = 3):
    import torch
    from qwen_triton_b200 import StepEntry
    engine = model.engine
    prompt = random_prompts(1, tokens, vocab, 11)[0]
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for it in range(warmup + repeats):
        slot = engine.new_sequence()
        torch.cuda.synchronize()
        begin.record()
        engine.step([StepEntry(slot, prompt, [tokens - 1])])
        end.record()
        torch.cuda.synchronize()
        engine.release(slot)
        if it >= warmup:
            times.append(begin.elapsed_time(end))
    return statistics.median(times)


def config_keys(preset: dict, args, layers: int) -> dict:
    """The flat description of the model and workload that both arms print."""
    return {
        "model": f"{args.preset} shape, random weights", "layers": layers, "layers_of_model": preset["num_hidden_layers"],
        "hidden": preset["hidden_size"], "heads": preset["num_attention_heads"], "kv_heads": preset["num_key_value_heads"],
        "head_dim": preset["head_dim"], "intermediate": preset["intermediate_size"], "vocab": preset["vocab_size"],
        "global_batch": args.batch, "prompt_len": args.prompt_len, "parallelism": "single_gpu",
        "steps_requested": args.steps, "min_seconds": args.min_seconds,
        "l2": "inputs larger than L2: every step streams all weights",
    }


def preset_json(name: str) -> dict:
    return json.loads((ROOT / "qwen_triton_b200" / "config" / "presets" / f"{name}.json").read_text())


MOST_STEPS = 1024        # a timed region never runs more steps than this (sizes the cache)


def run_b200(args) -> dict:
    import dataclasses

    from qwen_triton_b200 import QwenB200ForCausalLM, load_preset

    full = load_preset(args.preset)
    layers = args.layers or full.num_hidden_layers
    config = full if layers == full.num_hidden_layers else dataclasses.replace(
        full, num_hidden_layers=layers, layer_types=full.layer_types[:layers])
    peak, peak_source = peaks()
    numbers = model_numbers(config, layers)
    batches = [args.batch] if args.no_points else sorted({1, args.batch, 64})
    most_steps = max(args.steps, MOST_STEPS)
    max_context = -(-(args.prompt_len + args.warmup + most_steps + 16) // 64) * 64
    max_tokens = max(batches) * max_context + 4096
    model = QwenB200ForCausalLM.from_config(config, seed=0, dtype="bf16", max_tokens=max_tokens,
                                            max_seq_len=max_context, max_step_tokens=4096)
    vocab = config.vocab_size
    weight_bytes = 2 * (numbers["linear_params"] + numbers["head_params"])      # the embedding is read row-wise only

    from qwen_triton_b200.ops import kernels

    def progress(text: str) -> None:
        kernels.check_status(model.engine.device)        # raises if a bounded wait inside a kernel ran out
        print(f"[bench] {text}", file=sys.stderr, flush=True)

    def fraction(batch: int, result: dict) -> float:
        step_bytes = weight_bytes + batch * result["context"] * numbers["kv_bytes_per_token"]
        return step_bytes / (result["ms"] * 1e-3) / 1e9 / peak["hbm_gbs"]

    progress(f"model built: {layers} layers")
    results = {}
    for batch in batches:
        prompts = random_prompts(batch, args.prompt_len, vocab, 100 + batch)
        seconds = args.min_seconds if batch == args.batch else args.min_seconds / 2
        ms, launches, clocks, context, steps = time_decode(model, prompts, args.steps, args.warmup, vocab, seconds, most_steps)
        progress(f"decode at batch {batch}: {ms:.3f} ms per step over {steps} steps")
        results[batch] = {"ms": ms, "tok_s": batch * 1e3 / ms, "launches": launches, "clocks": clocks,
                          "context": context, "steps": steps}
    main = results[args.batch]
    step_bytes = weight_bytes + args.batch * main["context"] * numbers["kv_bytes_per_token"]
    achieved = step_bytes / (main["ms"] * 1e-3) / 1e9

    prompts = random_prompts(args.batch, args.prompt_len, vocab, 100 + args.batch)
    e2e_ms, h2d, d2h, e2e_steps = time_e2e(model, prompts, args.steps, args.warmup, args.min_seconds, most_steps, args.temperature)
    progress(f"end to end at batch {args.batch}: {e2e_ms:.3f} ms per step over {e2e_steps} steps")

    points = {}
    for batch, result in results.items():
        if batch != args.batch:
            points[f"decode_b{batch}"] = round(result["tok_s"], 2)
            points[f"decode_b{batch}_frac"] = round(fraction(batch, result), 4)
    line = {
        "metric": "decode_tokens_per_s", "value": round(main["tok_s"], 2), "unit": "tokens/s", "n_gpus": 1,
        "steps": main["steps"], "warmup": args.warmup, "ms_per_step": round(main["ms"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "b200",
        "config": {**config_keys(preset_json(args.preset), args, layers), "seq_len": args.prompt_len + args.warmup + main["steps"],
                   "context_mean": main["context"], "peaks": peak_source},
        "clocks": main["clocks"],
        "e2e": {"value": round(args.batch * 1e3 / e2e_ms, 2), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps, "temperature": args.temperature},
        "gpu_launches": main["launches"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4), "bytes_per_step": step_bytes},
        "points": points,
    }
    if not args.no_prefill:
        tokens = args.prompt_len
        ms = time_prefill(model, tokens, vocab)
        progress(f"prefill of {tokens} tokens: {ms:.3f} ms")
        flops = 2 * tokens * numbers["linear_params"] + 2 * numbers["head_params"] \
            + numbers["attn_flops_per_pair"] * tokens * (tokens + 1) // 2
        line["prefill"] = {"value": round(tokens * 1e3 / ms, 1), "tokens": tokens, "ms": round(ms, 3),
                           "frac": round(flops / (ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4), "flops": flops}
    return line


# ----------------------------------------------------------------------------- secondary workloads
def run_workload(args) -> dict:
    """BASELINE's secondary workloads as they are stated."""
    import torch

    from qwen_triton_b200 import QwenB200ForCausalLM, StepEntry, load_preset
    from qwen_triton_b200.ops import kernels

    peak, peak_source = peaks()
    if args.workload == "0.6b-unequal":
        config = load_preset("qwen3-0.6b")
        numbers = model_numbers(config, config.num_hidden_layers)
        generator = torch.Generator().manual_seed(16)
        lengths = torch.randint(64, 2049, (16,), generator=generator).tolist()
        prompts = [torch.randint(0, config.vocab_size, (n,), generator=generator).tolist() for n in lengths]
        new_tokens = 128
        model = QwenB200ForCausalLM.from_config(config, seed=0, dtype="bf16", max_tokens=16 * 2304 + 4096, max_seq_len=2304)
        times = []
        for _ in range(4):                                   # the first run warms up (launches, then captured steps)
            torch.cuda.synchronize()
            with ClockSampler() as clocks:
                start = time.perf_counter()
                results = model.generate(prompts, max_new_tokens=new_tokens, ignore_eos=True)
                torch.cuda.synchronize()
                times.append(time.perf_counter() - start)
        assert all(len(r.tokens) == new_tokens for r in results)
        seconds = statistics.median(times[1:])
        # decode alone, device-timed, from the same unequal caches
        engine = model.engine
        slots = [engine.new_sequence() for _ in prompts]
        for i in range(0, 16, 4):
            engine.step([StepEntry(slots[j], prompts[j], []) for j in range(i, i + 4)])
        out = torch.empty(16, dtype=torch.int32, device=engine.device)
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        feed = torch.randint(0, config.vocab_size, (8 + new_tokens, 16), generator=generator).tolist()
        for row in feed[:8]:
            kernels.argmax(engine.step([StepEntry(s, [t], [0]) for s, t in zip(slots, row)]), out)
        begin.record()
        for row in feed[8:]:
            kernels.argmax(engine.step([StepEntry(s, [t], [0]) for s, t in zip(slots, row)]), out)
        end.record()
        torch.cuda.synchronize()
        ms = begin.elapsed_time(end) / new_tokens
        weight_bytes = 2 * (numbers["linear_params"] + numbers["head_params"])
        step_bytes = weight_bytes + (sum(lengths) + 16 * (8 + new_tokens // 2)) * numbers["kv_bytes_per_token"]
        return {"workload": args.workload, "impl": "b200", "dtype": "bf16", "data": "synthetic",
                "config": {"model": "qwen3-0.6b shape, random weights", "layers": config.num_hidden_layers, "requests": 16,
                           "prompt_tokens": sum(lengths), "prompt_min": min(lengths), "prompt_max": max(lengths),
                           "new_tokens": new_tokens, "peaks": peak_source},
                "generate": {"seconds": round(seconds, 4), "new_tokens_per_s": round(16 * new_tokens / seconds, 1),
                             "all_tokens_per_s": round((sum(lengths) + 16 * new_tokens) / seconds, 1)},
                "decode": {"ms_per_step": round(ms, 4), "tokens_per_s": round(16e3 / ms, 1),
                           "frac": round(step_bytes / (ms * 1e-3) / 1e9 / peak["hbm_gbs"], 4), "bytes_per_step": step_bytes},
                "clocks": clocks.summary()}

    config = load_preset("qwen3-32b")
    numbers = model_numbers(config, config.num_hidden_layers)
    batch, first, last = 64, 2048, 4096
    model = QwenB200ForCausalLM.from_config(config, seed=0, dtype="bf16", max_tokens=batch * last + 4096, max_seq_len=last,
                                            max_step_tokens=4096)
    engine = model.engine
    print("[bench] model built", file=sys.stderr, flush=True)
    prompts = random_prompts(batch, first, config.vocab_size, 164)
    slots = [engine.new_sequence() for _ in prompts]
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for i in range(0, batch, 2):
        engine.step([StepEntry(slots[j], prompts[j], []) for j in range(i, i + 2)])
    end.record()
    torch.cuda.synchronize()
    prefill_ms = begin.elapsed_time(end)
    kernels.check_status(engine.device)
    print(f"[bench] prompts: {prefill_ms:.0f} ms", file=sys.stderr, flush=True)
    out = torch.zeros(batch, dtype=torch.int32, device=engine.device)
    weight_bytes = 2 * (numbers["linear_params"] + numbers["head_params"])
    marks, window = {}, 64
    # windows of 64 steps, clear of the first steps (launched, then captured) and of the context buckets' edges
    # (a new bucket's first two steps are launched and captured as well)
    centres = (first + 96, (first + last) // 2 - 64, last - 64)
    starts = {c - window // 2: c for c in centres}
    stops = {c + window // 2: c for c in centres}
    events = {c: [torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)] for c in centres}
    total_begin, total_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    rows = list(range(batch))
    with ClockSampler() as clocks:
        total_begin.record()
        for position in range(first, last):                  # the token fed at this step sits at `position`
            if position in starts:
                events[starts[position]][0].record()
            plan = engine.plan_decode(slots)
            if position == first:                            # the first tokens come from the host, the others stay on the device
                logits = engine.run_planned(plan, [p[-1] for p in prompts])
            else:
                logits = engine.run_planned(plan, rows, chosen=out)
            kernels.argmax(logits, out)
            if position + 1 in stops:
                events[stops[position + 1]][1].record()
        total_end.record()
        torch.cuda.synchronize()
    kernels.check_status(engine.device)
    total_ms = total_begin.elapsed_time(total_end)
    for centre, pair in events.items():
        ms = pair[0].elapsed_time(pair[1]) / window
        step_bytes = weight_bytes + batch * centre * numbers["kv_bytes_per_token"]
        marks[f"ctx_{centre}"] = {"ms_per_step": round(ms, 3), "tokens_per_s": round(batch * 1e3 / ms, 1),
                                  "frac": round(step_bytes / (ms * 1e-3) / 1e9 / peak["hbm_gbs"], 4)}
    return {"workload": args.workload, "impl": "b200", "dtype": "bf16", "data": "synthetic",
            "config": {"model": "qwen3-32b shape, random weights", "layers": config.num_hidden_layers, "global_batch": batch,
                       "from": first, "to": last, "peaks": peak_source},
            "prefill": {"tokens": batch * first, "ms": round(prefill_ms, 1), "tokens_per_s": round(batch * first * 1e3 / prefill_ms, 1)},
            "decode": {"steps": last - first, "seconds": round(total_ms / 1e3, 3),
                       "tokens_per_s": round(batch * (last - first) * 1e3 / total_ms, 1), **marks},
            "clocks": clocks.summary()}


# ----------------------------------------------------------------------------- the reference
def run_reference(args) -> dict:
    """The unmodified reference installed under baseline/_ref, through its own public API: build the model
    from the same configuration with random weights, prefill the batch with ``use_cache=True``, then time
    one-token forwards with ``logits_to_keep=1`` followed by argmax, as its ``greedy_generate`` does
    (qwen_triton/models/core.py:392-409).  ``value`` is timed on the device with the tokens given ahead; ``e2e``
    is that loop as the reference's generation runs it: token ids from the host to the device, forward, argmax,
    ids back to the host, every step, by the wall clock."""
    ref_root = ROOT / "baseline" / "_ref"
    if not (ref_root / "qwen_triton").exists():
        return {"impl": "reference", "unavailable": "baseline/_ref is not installed (pip install --target baseline/_ref of the reference)"}
    try:
        os.environ.setdefault("HF_HUB_OFFLINE", "1")
        sys.path.insert(0, str(ref_root))
        import torch
        from qwen_triton.configs import QwenTritonConfig
        from qwen_triton.models import QwenTritonForCausalLM

        preset = preset_json(args.preset)
        full_layers = preset["num_hidden_layers"]
        layers = args.layers or full_layers
        most_steps = max(args.steps, 256)
        preset["num_hidden_layers"] = layers
        preset["max_position_embeddings"] = -(-(args.prompt_len + 2 * (args.warmup + most_steps) + 8) // 64) * 64
        torch.manual_seed(0)
        with torch.device("cuda"):
            model = QwenTritonForCausalLM.from_config(QwenTritonConfig.from_hf_config(preset))
        model = model.to(torch.bfloat16).eval()
        vocab = preset["vocab_size"]
        ids = torch.tensor(random_prompts(args.batch, args.prompt_len, vocab, 100 + args.batch), device="cuda")
        generator = torch.Generator().manual_seed(7)
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.no_grad():
            out = model(input_ids=ids, use_cache=True, logits_to_keep=1)
            cache = out.past_key_values

            def one(tokens):
                nonlocal cache
                step = model(input_ids=tokens, past_key_values=cache, use_cache=True, logits_to_keep=1)
                cache = step.past_key_values
                return step.logits[:, -1].argmax(dim=-1)

            feed = torch.randint(0, vocab, (args.warmup, args.batch, 1), generator=generator).cuda()
            torch.cuda.synchronize()
            begin.record()
            for t in range(args.warmup):
                one(feed[t])
            end.record()
            torch.cuda.synchronize()
            steps = steps_for(begin.elapsed_time(end) / max(1, args.warmup), args.steps, args.min_seconds, most_steps)
            feed = torch.randint(0, vocab, (steps, args.batch, 1), generator=generator).cuda()
            with ClockSampler() as clocks:
                begin.record()
                for t in range(steps):
                    one(feed[t])
                end.record()
                torch.cuda.synchronize()
            ms = begin.elapsed_time(end) / steps

            # end to end: the last tokens go from the host to the device, the chosen ones come back, every step
            e2e_steps = steps_for(ms, args.steps, args.min_seconds, most_steps)
            host = torch.randint(0, vocab, (args.batch, 1), generator=generator).pin_memory()
            back = torch.empty(args.batch, dtype=torch.long).pin_memory()
            torch.cuda.synchronize()
            wall = time.perf_counter()
            for _ in range(e2e_steps):
                chosen = one(host.to("cuda", non_blocking=True))
                back.copy_(chosen, non_blocking=True)
                torch.cuda.synchronize()
                host.copy_(back[:, None])
            e2e_ms = (time.perf_counter() - wall) * 1e3 / e2e_steps
        return {
            "metric": "decode_tokens_per_s", "value": round(args.batch * 1e3 / ms, 2), "unit": "tokens/s", "n_gpus": 1,
            "steps": steps, "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
            "config": {**config_keys(preset_json(args.preset), args, layers), "seq_len": args.prompt_len + args.warmup + steps,
                       "context_mean": args.prompt_len + args.warmup + steps // 2},
            "clocks": clocks.summary(),
            "e2e": {"value": round(args.batch * 1e3 / e2e_ms, 2), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                    "h2d_bytes_per_step": 8 * args.batch, "d2h_bytes_per_step": 8 * args.batch, "steps": e2e_steps},
        }
    except Exception as exc:  # the reference could not run here: say why in one line
        return {"impl": "reference", "unavailable": f"{type(exc).__name__}: {str(exc).splitlines()[0][:200] if str(exc) else ''}"}


def main() -> int:
    args = parse_args()
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not measured")
        return 2
    if args.workload:
        if args.impl == "reference":
            line = {"impl": "reference", "workload": args.workload,
                    "unavailable": "the secondary workloads are measured for this library only (the reference has no generation benchmark)"}
        else:
            line = run_workload(args)
    else:
        line = run_reference(args) if args.impl == "reference" else run_b200(args)
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
