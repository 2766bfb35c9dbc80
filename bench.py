"""Decode and prefill throughput of the Qwen3-8B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl b200|reference]

Prints ONE JSON line.  ``value`` is decoded tokens per second at batch 8 from a 2,048-token cache,
timed on the device over K decode steps (step function plus greedy sampling kernel, tokens given
ahead); ``e2e`` is the same through the Python entry point with host token ids in and out at every
step; ``prefill`` is one 2,048-token prompt; ``roofline`` is the decode step's bytes (every weight
once plus the live cache) over its time against the measured HBM copy bandwidth; ``points`` holds
batch 1 and 64.  Weights are random, token ids are uniform random with a fixed seed.
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


def time_decode(model, prompts, steps: int, warmup: int, vocab: int):
    """Device-timed decode: the batch's cache is filled by a real prefill, then ``warmup`` + ``steps`` steps of
    one given token per sequence, each followed by the greedy sampling kernel."""
    import torch
    from qwen_triton_b200 import StepEntry
    from qwen_triton_b200.ops import kernels

    engine = model.engine
    slots = [engine.new_sequence() for _ in prompts]
    for start in range(0, len(prompts), 2):      # fill the cache two prompts at a time
        part = range(start, min(start + 2, len(prompts)))
        engine.step([StepEntry(slots[i], prompts[i], []) for i in part])
    generator = torch.Generator().manual_seed(7)
    feed = torch.randint(0, vocab, (warmup + steps, len(prompts)), generator=generator).tolist()
    out = torch.empty(len(prompts), dtype=torch.int32, device=engine.device)
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def one(tokens):
        logits = engine.step([StepEntry(slot, [tok], [0]) for slot, tok in zip(slots, tokens)])
        kernels.argmax(logits, out)

    for tokens in feed[:warmup]:
        one(tokens)
    torch.cuda.synchronize()
    launches = kernels.launch_count()
    with ClockSampler() as clocks:
        begin.record()
        for tokens in feed[warmup:]:
            one(tokens)
        end.record()
        torch.cuda.synchronize()
    launches = kernels.launch_count() - launches
    ms = begin.elapsed_time(end) / steps
    context = len(prompts[0]) + warmup + steps // 2          # mean cache length during the timed steps
    for slot in slots:
        engine.release(slot)
    return ms, launches, clocks.summary(), context


def time_e2e(model, prompts, steps: int, warmup: int):
    """Through the entry point: host token ids in, sampled token ids back on the host, every step."""
    import torch
    run = model.start_batch(prompts, max_new_tokens=warmup + steps + 1, ignore_eos=True)
    run.start()
    for _ in range(warmup):
        run.advance()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall = time.perf_counter()
    begin.record()
    for _ in range(steps):
        run.advance()
    end.record()
    torch.cuda.synchronize()
    wall = (time.perf_counter() - wall) * 1e3 / steps
    ms = max(begin.elapsed_time(end) / steps, wall)
    h2d = model.engine.last_meta_bytes
    run.close()
    return ms, h2d, 4 * len(prompts)


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


def run_b200(args) -> dict:
    import dataclasses

    import torch

    from qwen_triton_b200 import QwenB200ForCausalLM, load_preset

    full = load_preset(args.preset)
    layers = args.layers or full.num_hidden_layers
    config = full if layers == full.num_hidden_layers else dataclasses.replace(
        full, num_hidden_layers=layers, layer_types=full.layer_types[:layers])
    peak, peak_source = peaks()
    numbers = model_numbers(config, layers)
    batches = [args.batch] if args.no_points else sorted({1, args.batch, 64})
    total_steps = args.steps + args.warmup + 2
    max_context = args.prompt_len + 2 * total_steps
    max_tokens = max(batches) * (-(-max_context // 64) * 64) + 4096
    model = QwenB200ForCausalLM.from_config(config, seed=0, dtype="bf16", max_tokens=max_tokens,
                                            max_seq_len=-(-max_context // 64) * 64, max_step_tokens=4096)
    vocab = config.vocab_size
    weight_bytes = 2 * (numbers["linear_params"] + numbers["head_params"])      # the embedding is read row-wise only

    from qwen_triton_b200.ops import kernels

    def progress(text: str) -> None:
        kernels.check_status(model.engine.device)        # raises if a bounded wait inside a kernel ran out
        print(f"[bench] {text}", file=sys.stderr, flush=True)

    progress(f"model built: {layers} layers")
    results = {}
    for batch in batches:
        prompts = random_prompts(batch, args.prompt_len, vocab, 100 + batch)
        steps = args.steps if batch == args.batch else max(8, args.steps // 4)
        ms, launches, clocks, context = time_decode(model, prompts, steps, args.warmup, vocab)
        progress(f"decode at batch {batch}: {ms:.3f} ms per step")
        results[batch] = {"ms": ms, "tok_s": batch * 1e3 / ms, "launches": launches, "clocks": clocks,
                          "context": context, "steps": steps}
    main = results[args.batch]
    step_bytes = weight_bytes + args.batch * main["context"] * numbers["kv_bytes_per_token"]
    achieved = step_bytes / (main["ms"] * 1e-3) / 1e9

    prompts = random_prompts(args.batch, args.prompt_len, vocab, 100 + args.batch)
    e2e_ms, h2d, d2h = time_e2e(model, prompts, args.steps, args.warmup)
    progress(f"end to end at batch {args.batch}: {e2e_ms:.3f} ms per step")

    line = {
        "metric": "decode_tokens_per_s", "value": round(main["tok_s"], 2), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(main["ms"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "b200",
        "config": {
            "model": f"{args.preset} shape, random weights", "layers": layers, "layers_of_model": full.num_hidden_layers,
            "hidden": config.hidden_size, "heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads,
            "head_dim": config.head_dim, "intermediate": config.intermediate_size, "vocab": vocab,
            "global_batch": args.batch, "seq_len": args.prompt_len + args.warmup + args.steps,
            "prompt_len": args.prompt_len, "context_mean": main["context"], "parallelism": "single_gpu",
            "l2": "inputs larger than L2: every step streams all weights", "peaks": peak_source,
        },
        "clocks": main["clocks"],
        "e2e": {"value": round(args.batch * 1e3 / e2e_ms, 2), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": main["launches"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4), "bytes_per_step": step_bytes},
        "points": {f"decode_b{b}": round(r["tok_s"], 2) for b, r in results.items() if b != args.batch},
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


# ----------------------------------------------------------------------------- the reference
def run_reference(args) -> dict:
    """The unmodified reference installed under baseline/_ref, through its own public API: build the model
    from the same configuration with random weights, prefill the batch with ``use_cache=True``, then time
    one-token forwards with ``logits_to_keep=1`` followed by argmax, as its ``greedy_generate`` does."""
    ref_root = ROOT / "baseline" / "_ref"
    if not (ref_root / "qwen_triton").exists():
        return {"impl": "reference", "unavailable": "baseline/_ref is not installed (pip install --target baseline/_ref of the reference)"}
    try:
        os.environ.setdefault("HF_HUB_OFFLINE", "1")
        sys.path.insert(0, str(ref_root))
        import torch
        from qwen_triton.configs import QwenTritonConfig
        from qwen_triton.models import QwenTritonForCausalLM

        preset = json.loads((ROOT / "qwen_triton_b200" / "config" / "presets" / f"{args.preset}.json").read_text())
        layers = args.layers or preset["num_hidden_layers"]
        preset["num_hidden_layers"] = layers
        preset["max_position_embeddings"] = 4096
        torch.manual_seed(0)
        with torch.device("cuda"):
            model = QwenTritonForCausalLM.from_config(QwenTritonConfig.from_hf_config(preset))
        model = model.to(torch.bfloat16).eval()
        vocab = preset["vocab_size"]
        ids = torch.tensor(random_prompts(args.batch, args.prompt_len, vocab, 100 + args.batch), device="cuda")
        generator = torch.Generator().manual_seed(7)
        feed = torch.randint(0, vocab, (args.warmup + args.steps, args.batch, 1), generator=generator).cuda()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.no_grad():
            out = model(input_ids=ids, use_cache=True, logits_to_keep=1)
            cache = out.past_key_values

            def one(tokens):
                nonlocal cache
                step = model(input_ids=tokens, past_key_values=cache, use_cache=True, logits_to_keep=1)
                cache = step.past_key_values
                return step.logits[:, -1].argmax(dim=-1)

            for t in range(args.warmup):
                one(feed[t])
            torch.cuda.synchronize()
            with ClockSampler() as clocks:
                begin.record()
                for t in range(args.warmup, args.warmup + args.steps):
                    one(feed[t])
                end.record()
                torch.cuda.synchronize()
        ms = begin.elapsed_time(end) / args.steps
        return {
            "metric": "decode_tokens_per_s", "value": round(args.batch * 1e3 / ms, 2), "unit": "tokens/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
            "config": {"model": f"{args.preset} shape, random weights", "layers": layers,
                       "layers_of_model": json.loads((ROOT / "qwen_triton_b200" / "config" / "presets" / f"{args.preset}.json").read_text())["num_hidden_layers"],
                       "global_batch": args.batch, "seq_len": args.prompt_len + args.warmup + args.steps,
                       "prompt_len": args.prompt_len, "parallelism": "single_gpu"},
            "clocks": clocks.summary(),
        }
    except Exception as exc:  # the reference could not run here: say why in one line
        return {"impl": "reference", "unavailable": f"{type(exc).__name__}: {str(exc).splitlines()[0][:200] if str(exc) else ''}"}


def main() -> int:
    args = parse_args()
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not measured")
        return 2
    line = run_reference(args) if args.impl == "reference" else run_b200(args)
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
