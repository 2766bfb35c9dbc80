"""Run a few steps of one workload, for profilers and launch lists (the reference has
``qwen_triton/scripts/profile_backend_step.py`` for its train/eval step).

    python -m qwen_triton_b200.scripts.profile_step --mode decode --batch 8 --context 2048 --layers 4
    python -m qwen_triton_b200.scripts.profile_step --mode prefill --tokens 2048 --layers 4
    python -m qwen_triton_b200.scripts.profile_step --mode sampling --batch 8 --top-p 0.9

Random weights of the given preset (optionally fewer layers, to keep a capture small), random token
ids.  Prints the mean step time measured with CUDA events; under a profiler that number is not a
benchmark value.
"""
from __future__ import annotations

import argparse
import dataclasses


def main(argv=None) -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--preset", default="qwen3-8b")
    parser.add_argument("--mode", choices=["decode", "prefill", "sampling"], default="decode",
                        help="'sampling': the choice of the next token alone, on random logits of the preset's vocabulary")
    parser.add_argument("--temperature", type=float, default=0.8)
    parser.add_argument("--top-k", type=int, default=0)
    parser.add_argument("--top-p", type=float, default=1.0)
    parser.add_argument("--dtype", default="bf16")
    parser.add_argument("--layers", type=int, default=0)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=2048, help="cache length before the decode steps")
    parser.add_argument("--tokens", type=int, default=2048, help="prompt length of the prefill step")
    parser.add_argument("--steps", type=int, default=3)
    parser.add_argument("--warmup", type=int, default=2)
    parser.add_argument("--fill", choices=["prefill", "skip"], default="prefill",
                        help="'skip' leaves the cache content as allocated (zeros): same work for a decode step, no prefill launches")
    parser.add_argument("--no-graphs", action="store_true", help="launch every kernel of a decode step (no CUDA graph replay)")
    args = parser.parse_args(argv)

    import torch
    from qwen_triton_b200 import QwenB200ForCausalLM, StepEntry, load_preset

    full = load_preset(args.preset)
    if args.mode == "sampling":
        from qwen_triton_b200.ops import kernels
        generator = torch.Generator(device="cuda").manual_seed(3)
        logits = torch.randn(args.batch, full.vocab_size, generator=generator, device="cuda") * 2.5
        keys = torch.stack([torch.arange(args.batch), torch.zeros(args.batch, dtype=torch.long)], dim=1).int().cuda()
        out = torch.empty(args.batch, dtype=torch.int32, device="cuda")
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for name, run in (("argmax", lambda: kernels.argmax(logits, out)),
                          (f"temperature {args.temperature}, top_k {args.top_k}, top_p {args.top_p}",
                           lambda: kernels.sample_keyed(logits, args.temperature, 1, keys, out, args.top_k, args.top_p))):
            for _ in range(args.warmup):
                run()
            torch.cuda.synchronize()
            begin.record()
            for _ in range(args.steps):
                run()
            end.record()
            torch.cuda.synchronize()
            print(f"{name}: {begin.elapsed_time(end) / args.steps * 1e3:.1f} us for {args.batch} rows of {full.vocab_size}")
        return
    layers = args.layers or full.num_hidden_layers
    config = dataclasses.replace(full, num_hidden_layers=layers, layer_types=full.layer_types[:layers])
    span = (args.context if args.mode == "decode" else args.tokens) + args.steps + args.warmup + 64
    span = -(-span // 64) * 64
    model = QwenB200ForCausalLM.from_config(config, seed=0, dtype=args.dtype, max_tokens=args.batch * span + 4096,
                                            max_seq_len=span, max_step_tokens=4096, cuda_graphs=not args.no_graphs)
    engine = model.engine
    generator = torch.Generator().manual_seed(3)
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    if args.mode == "prefill":
        prompt = torch.randint(0, config.vocab_size, (args.tokens,), generator=generator).tolist()
        times = []
        for it in range(args.warmup + args.steps):
            slot = engine.new_sequence()
            torch.cuda.synchronize()
            begin.record()
            engine.step([StepEntry(slot, prompt, [args.tokens - 1])])
            end.record()
            torch.cuda.synchronize()
            engine.release(slot)
            if it >= args.warmup:
                times.append(begin.elapsed_time(end))
        print(f"prefill of {args.tokens} tokens, {layers} layers: {sum(times) / len(times):.3f} ms")
        return

    slots = [engine.new_sequence() for _ in range(args.batch)]
    if args.fill == "prefill":
        for slot in slots:
            prompt = torch.randint(0, config.vocab_size, (args.context,), generator=generator).tolist()
            engine.step([StepEntry(slot, prompt, [])])
    else:
        for slot in slots:
            engine.cache.book.extend(slot, args.context)
    feed = torch.randint(0, config.vocab_size, (args.warmup + args.steps, args.batch), generator=generator).tolist()
    for tokens in feed[:args.warmup]:
        engine.step([StepEntry(s, [t], [0]) for s, t in zip(slots, tokens)])
    torch.cuda.synchronize()
    begin.record()
    for tokens in feed[args.warmup:]:
        engine.step([StepEntry(s, [t], [0]) for s, t in zip(slots, tokens)])
    end.record()
    torch.cuda.synchronize()
    print(f"decode at batch {args.batch}, context {args.context}, {layers} layers: "
          f"{begin.elapsed_time(end) / args.steps:.3f} ms per step")


if __name__ == "__main__":
    main()
