"""Command line in the manner of the reference's ``python -m qwen_triton.scripts.smoke``
(qwen_triton/scripts/smoke.py:12-72): load a model, run one forward, generate, print.

Options the reference has keep their names and meanings: ``--model-id``, ``--backend``,
``--device``, ``--dtype``, ``--prompt``, ``--max-new-tokens``, ``--compare-ref``.  ``--compare-ref``
compares the logits with the library's own true-float32 path on the same weights (the reference
compares with the upstream model class, which this library does not import).  ``--strict-triton`` is
accepted and has no effect: every kernel failure raises here.

Added: a model without a folder (``--preset NAME --random-weights``), prompts as token ids
(``--prompt-ids 1,2,3``, repeatable: a batch of unequal prompts) or random (``--random-prompts 5,9,17``),
``--temperature``, ``--seed`` (the seed of everything the run draws: sampling, random weights, random
prompts; ``--sampling-seed`` and ``--weights-seed`` set one of them apart), ``--stop-ids``,
``--ignore-eos``, ``--max-tokens`` (cache size), ``--max-seq-len``, ``--max-batch-size``.
"""
from __future__ import annotations

import argparse
from pathlib import Path


def _parse_args(argv=None) -> argparse.Namespace:
    parser = argparse.ArgumentParser(description="qwen_triton_b200 smoke run")
    parser.add_argument("--model-id", default=None, help="local model folder (config.json + safetensors)")
    parser.add_argument("--preset", default=None, help="name of a configuration shipped with the package (with --random-weights)")
    parser.add_argument("--random-weights", action="store_true", help="draw the weights from --seed instead of reading a folder")
    parser.add_argument("--backend", default="b200", choices=["b200"])
    parser.add_argument("--device", default="cuda:0")
    parser.add_argument("--dtype", default="bf16")
    parser.add_argument("--prompt", default=None, help="text prompt; needs tokenizer.json in the model folder")
    parser.add_argument("--prompt-ids", action="append", default=None,
                        help="comma-separated token ids; repeat for a batch of unequal prompts")
    parser.add_argument("--random-prompts", default=None, help="comma-separated lengths of prompts of uniform random token ids")
    parser.add_argument("--max-new-tokens", type=int, default=8)
    parser.add_argument("--temperature", type=float, default=0.0)
    parser.add_argument("--top-k", type=int, default=0, help="with --temperature: draw from the k most likely tokens only")
    parser.add_argument("--top-p", type=float, default=1.0, help="with --temperature: draw from the most likely tokens that sum to this share")
    parser.add_argument("--seed", type=int, default=0, help="seed of everything the run draws")
    parser.add_argument("--sampling-seed", type=int, default=None, help="seed of temperature sampling (default: --seed)")
    parser.add_argument("--weights-seed", type=int, default=None, help="seed of --random-weights (default: --seed)")
    parser.add_argument("--stop-ids", default="", help="comma-separated extra stop token ids")
    parser.add_argument("--ignore-eos", action="store_true")
    parser.add_argument("--max-tokens", type=int, default=8192, help="cache size in tokens")
    parser.add_argument("--max-seq-len", type=int, default=None, help="longest sequence (prompt and new tokens) the cache holds")
    parser.add_argument("--max-batch-size", type=int, default=None, help="most requests that run as one batch")
    parser.add_argument("--compare-ref", action="store_true")
    parser.add_argument("--strict-triton", action="store_true")
    args = parser.parse_args(argv)
    if args.random_weights != (args.preset is not None) or (args.model_id is None) == (args.preset is None):
        parser.error("give either --model-id FOLDER or --preset NAME --random-weights")
    given = sum(x is not None for x in (args.prompt, args.prompt_ids, args.random_prompts))
    if given > 1:
        parser.error("give one of --prompt, --prompt-ids and --random-prompts")
    return args


def _ids(text: str, what: str) -> list[int]:
    try:
        return [int(t) for t in text.split(",") if t.strip()]
    except ValueError:
        raise SystemExit(f"{what}: {text!r} is not a comma-separated list of integers") from None


def _load_tokenizer(model_dir: Path | None):
    path = None if model_dir is None else model_dir / "tokenizer.json"
    if path is None or not path.exists():
        raise SystemExit("--prompt needs tokenizer.json in a model folder; pass --prompt-ids or --random-prompts instead")
    from tokenizers import Tokenizer
    return Tokenizer.from_file(str(path))


def main(argv=None) -> None:
    args = _parse_args(argv)
    import torch
    from qwen_triton_b200 import QwenB200ForCausalLM, load_preset

    options = {"max_tokens": args.max_tokens}
    if args.max_seq_len is not None:
        options["max_seq_len"] = args.max_seq_len
    weights_seed = args.seed if args.weights_seed is None else args.weights_seed
    sampling_seed = args.seed if args.sampling_seed is None else args.sampling_seed

    def build(dtype: str):
        """The model in ``dtype``; with random weights, always the values a bfloat16 folder of --dtype would hold."""
        if args.random_weights:
            return QwenB200ForCausalLM.from_config(load_preset(args.preset), seed=weights_seed, device=args.device,
                                                   dtype=dtype, weights_dtype=args.dtype, **options)
        return QwenB200ForCausalLM.from_pretrained_hf(args.model_id, backend=args.backend, device=args.device,
                                                      dtype=dtype, **options)

    model = build(args.dtype)
    vocab = model.engine.vocab_size
    tokenizer = None
    if args.prompt_ids:
        prompts = [_ids(item, "--prompt-ids") for item in args.prompt_ids]
    elif args.random_prompts:
        generator = torch.Generator().manual_seed(args.seed)
        prompts = [torch.randint(0, vocab, (n,), generator=generator).tolist() for n in _ids(args.random_prompts, "--random-prompts")]
    else:
        tokenizer = _load_tokenizer(Path(args.model_id) if args.model_id else None)
        prompts = [tokenizer.encode(args.prompt or "Write one sentence about GPU kernels.").ids]
    if not prompts or any(not p for p in prompts):
        raise SystemExit("every prompt needs at least one token")

    outputs = model.forward(prompts[0], logits_to_keep=1)
    next_token = outputs.logits[:, -1].argmax(dim=-1)
    results = model.generate(prompts, max_new_tokens=args.max_new_tokens, temperature=args.temperature,
                             seed=sampling_seed, stop_token_ids=_ids(args.stop_ids, "--stop-ids"),
                             ignore_eos=args.ignore_eos, max_batch_size=args.max_batch_size, top_k=args.top_k, top_p=args.top_p)
    print(f"backend={args.backend}")
    print(f"next_token={next_token.tolist()}")
    for prompt, result in zip(prompts, results):
        if tokenizer is not None:
            print(tokenizer.decode(prompt + result.tokens))
        else:
            print(f"generated={result.tokens} finish={result.finish_reason}")

    if args.compare_ref:
        kept = outputs.logits.float().cpu()
        del model, outputs
        torch.cuda.empty_cache()
        ref_logits = build("fp32").forward(prompts[0], logits_to_keep=1).logits.float().cpu()
        diff = (kept - ref_logits).abs()
        print(f"logit_max_abs_diff={float(diff.max()):.6f}")
        print(f"logit_mean_abs_diff={float(diff.mean()):.6f}")


if __name__ == "__main__":
    main()
