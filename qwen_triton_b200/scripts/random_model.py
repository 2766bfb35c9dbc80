"""Write a model folder (config.json, model.safetensors) with seeded random weights.

    python -m qwen_triton_b200.scripts.random_model --preset tiny-a --seed 0 --dtype fp32 --out DIR
    python -m qwen_triton_b200.scripts.random_model --config path/to/config.json --out DIR
"""
from __future__ import annotations

import argparse


def main(argv=None) -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    group = parser.add_mutually_exclusive_group(required=True)
    group.add_argument("--preset", help="name of a configuration shipped with the package")
    group.add_argument("--config", help="a config.json (or a folder holding one)")
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--dtype", default="bf16")
    parser.add_argument("--out", required=True)
    args = parser.parse_args(argv)

    from qwen_triton_b200.config import load_config, load_preset
    from qwen_triton_b200.engine import parse_dtype
    from qwen_triton_b200.weights import write_random_model

    config = load_preset(args.preset) if args.preset else load_config(args.config)
    folder = write_random_model(args.out, config, args.seed, parse_dtype(args.dtype))
    print(folder)


if __name__ == "__main__":
    main()
