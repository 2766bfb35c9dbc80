"""Command line in the manner of the reference's ``python -m qwen_triton.scripts.smoke``
(qwen_triton/scripts/smoke.py:12-72): load a model folder, run one forward, generate, print.

Options the reference has keep their names and meanings: ``--model-id``, ``--backend``,
``--device``, ``--dtype``, ``--prompt``, ``--max-new-tokens``, ``--compare-ref``.  ``--compare-ref``
compares the logits with the library's own true-float32 path (the reference compares with the
upstream model class, which this library does not import).  ``--strict-triton`` is accepted and
has no effect: every kernel failure raises here.  Added: ``--prompt-ids``, ``--temperature``,
``--seed``, ``--stop-ids``, ``--ignore-eos``, ``--max-tokens``.
"""
from __future__ import annotations

import argparse
from pathlib import Path


def _parse_args(argv=None) -> argparse.Namespace:
    parser = argparse.ArgumentParser(description="qwen_triton_b200 smoke run")
    parser.add_argument("--model-id", required=True, help="local model folder (config.json + safetensors)")
    parser.add_argument("--backend", default="b200", choices=["b200"])
    parser.add_argument("--device", default="cuda:0")
    parser.add_argument("--dtype", default="bf16")
    parser.add_argument("--prompt", default=None, help="text prompt; needs tokenizer.json in the model folder")
    parser.add_argument("--prompt-ids", action="append", default=None,
                        help="comma-separated token ids; repeat for a batch of unequal prompts")
    parser.add_argument("--max-new-tokens", type=int, default=8)
    parser.add_argument("--temperature", type=float, default=0.0)
    parser.add_argument("--seed", type=int, default=0, help="sampling seed")
    parser.add_argument("--stop-ids", default="", help="comma-separated extra stop token ids")
    parser.add_argument("--ignore-eos", action="store_true")
    parser.add_argument("--max-tokens", type=int, default=8192, help="cache size in tokens")
    parser.add_argument("--compare-ref", action="store_true")
    parser.add_argument("--strict-triton", action="store_true")
    return parser.parse_args(argv)


def _load_tokenizer(model_dir: Path):
    path = model_dir / "tokenizer.json"
    if not path.exists():
        raise SystemExit(f"--prompt needs {path}; pass --prompt-ids instead")
    from tokenizers import Tokenizer
    return Tokenizer.from_file(str(path))


def main(argv=None) -> None:
    args = _parse_args(argv)
    import torch
    from qwen_triton_b200 import QwenB200ForCausalLM

    model_dir = Path(args.model_id)
    tokenizer = None
    if args.prompt_ids:
        prompts = [[int(t) for t in item.split(",") if t.strip()] for item in args.prompt_ids]
    else:
        tokenizer = _load_tokenizer(model_dir)
        prompts = [tokenizer.encode(args.prompt or "Write one sentence about GPU kernels.").ids]

    model = QwenB200ForCausalLM.from_pretrained_hf(args.model_id, backend=args.backend, device=args.device,
                                                   dtype=args.dtype, max_tokens=args.max_tokens)
    outputs = model.forward(prompts[0], logits_to_keep=1)
    next_token = outputs.logits[:, -1].argmax(dim=-1)
    stop_ids = [int(t) for t in args.stop_ids.split(",") if t.strip()]
    results = model.generate(prompts, max_new_tokens=args.max_new_tokens, temperature=args.temperature,
                             seed=args.seed, stop_token_ids=stop_ids, ignore_eos=args.ignore_eos)
    print(f"backend={args.backend}")
    print(f"next_token={next_token.tolist()}")
    for prompt, result in zip(prompts, results):
        if tokenizer is not None:
            print(tokenizer.decode(prompt + result.tokens))
        else:
            print(f"generated={result.tokens} finish={result.finish_reason}")

    if args.compare_ref:
        del model
        torch.cuda.empty_cache()
        ref = QwenB200ForCausalLM.from_pretrained_hf(args.model_id, device=args.device, dtype="fp32",
                                                     max_tokens=args.max_tokens)
        ref_logits = ref.forward(prompts[0], logits_to_keep=1).logits
        diff = (outputs.logits.float() - ref_logits.float()).abs()
        print(f"logit_max_abs_diff={float(diff.max()):.6f}")
        print(f"logit_mean_abs_diff={float(diff.mean()):.6f}")


if __name__ == "__main__":
    main()
