"""Run luozoupi/Qwen-Triton's own model code on the CPU and store its logits.

Usage:  QWEN_TRITON_REFERENCE=/path/to/Qwen-Triton python tests/golden/make_golden.py

For each tiny configuration below the script builds the reference's
``QwenTritonForCausalLM`` (qwen_triton/models/core.py:250-293) on the CPU in
float32, where every kernel takes its torch formula, fills it with the weights
of :func:`golden_weights`, and stores in ``<name>.npz``: the prompt, the logits
of the whole prompt in one forward without cache, and a greedy continuation
from ``greedy_generate`` (core.py:377-409).  For the windowed configuration the
continuation is instead the argmax of repeated whole forwards without cache:
the reference's cached decode branch drops the mask and with it the window
(qwen_triton/modules/attention.py:100-109), while its whole forward applies it
(core.py:211-219), and the window rule is what is checked here.  Weights are not stored; the test
draws them again with the same recipe.  The reference is imported from the
given path and left unchanged.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent

CONFIGS = {
    "golden_a": dict(model_type="qwen3", vocab_size=256, hidden_size=64, intermediate_size=128,
                     num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                     rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                     max_position_embeddings=128),
    "golden_b": dict(model_type="qwen3", vocab_size=503, hidden_size=96, intermediate_size=160,
                     num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=1, head_dim=32,
                     rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
                     max_position_embeddings=128),
    "golden_c": dict(model_type="qwen3", vocab_size=311, hidden_size=80, intermediate_size=112,
                     num_hidden_layers=4, num_attention_heads=6, num_key_value_heads=3, head_dim=48,
                     rope_theta=50000.0, rms_norm_eps=3e-6, tie_word_embeddings=False,
                     max_position_embeddings=128, use_sliding_window=True, sliding_window=5,
                     max_window_layers=2),
    "golden_d": dict(model_type="qwen3", vocab_size=199, hidden_size=72, intermediate_size=88,
                     num_hidden_layers=2, num_attention_heads=3, num_key_value_heads=3, head_dim=32,
                     rope_theta=20000.0, rms_norm_eps=2e-6, tie_word_embeddings=True,
                     max_position_embeddings=128, attention_bias=True),
}
PROMPT_LENGTHS = {"golden_a": 17, "golden_b": 31, "golden_c": 23, "golden_d": 19}
SEEDS = {"golden_a": 0, "golden_b": 1, "golden_c": 2, "golden_d": 3}
GREEDY_PROMPT = 6
GREEDY_NEW = 5


def tensor_names(raw: dict) -> list[str]:
    names = ["model.embed_tokens.weight", "model.norm.weight"]
    if not raw["tie_word_embeddings"]:
        names.append("lm_head.weight")
    for i in range(raw["num_hidden_layers"]):
        p = f"model.layers.{i}"
        names += [f"{p}.input_layernorm.weight", f"{p}.post_attention_layernorm.weight",
                  f"{p}.self_attn.q_proj.weight", f"{p}.self_attn.k_proj.weight", f"{p}.self_attn.v_proj.weight",
                  f"{p}.self_attn.o_proj.weight", f"{p}.self_attn.q_norm.weight", f"{p}.self_attn.k_norm.weight",
                  f"{p}.mlp.gate_proj.weight", f"{p}.mlp.up_proj.weight", f"{p}.mlp.down_proj.weight"]
        if raw.get("attention_bias"):
            names += [f"{p}.self_attn.{proj}.bias" for proj in ("q_proj", "k_proj", "v_proj", "o_proj")]
    return sorted(names)


def tensor_shape(raw: dict, name: str) -> tuple[int, ...]:
    h, d = raw["hidden_size"], raw["head_dim"]
    nq, nkv, inter, vocab = raw["num_attention_heads"], raw["num_key_value_heads"], raw["intermediate_size"], raw["vocab_size"]
    leaf = name.split(".")[-2]
    if name.endswith(".bias"):
        return {"q_proj": (nq * d,), "k_proj": (nkv * d,), "v_proj": (nkv * d,), "o_proj": (h,)}[leaf]
    return {
        "embed_tokens": (vocab, h), "lm_head": (vocab, h), "norm": (h,),
        "input_layernorm": (h,), "post_attention_layernorm": (h,),
        "q_proj": (nq * d, h), "k_proj": (nkv * d, h), "v_proj": (nkv * d, h), "o_proj": (h, nq * d),
        "q_norm": (d,), "k_norm": (d,),
        "gate_proj": (inter, h), "up_proj": (inter, h), "down_proj": (h, inter),
    }[leaf]


def golden_weights(raw: dict, seed: int) -> dict[str, torch.Tensor]:
    """Matrices N(0, 0.05), norm weights 1 + N(0, 0.2), biases N(0, 0.2); one generator per tensor."""
    out = {}
    for index, name in enumerate(tensor_names(raw)):
        generator = torch.Generator().manual_seed(seed * 1000 + index)
        shape = tensor_shape(raw, name)
        values = torch.randn(shape, generator=generator, dtype=torch.float32)
        out[name] = 0.2 * values if name.endswith(".bias") else 1.0 + 0.2 * values if len(shape) == 1 else 0.05 * values
    return out


def golden_prompt(name: str) -> list[int]:
    generator = torch.Generator().manual_seed(100 + SEEDS[name])
    return torch.randint(0, CONFIGS[name]["vocab_size"], (PROMPT_LENGTHS[name],), generator=generator).tolist()


def main() -> None:
    reference = os.environ.get("QWEN_TRITON_REFERENCE")
    if not reference:
        raise SystemExit("set QWEN_TRITON_REFERENCE to a checkout of luozoupi/Qwen-Triton")
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    sys.path.insert(0, reference)
    from qwen_triton.configs import QwenTritonConfig
    from qwen_triton.models import QwenTritonForCausalLM

    for name, raw in CONFIGS.items():
        model = QwenTritonForCausalLM.from_config(QwenTritonConfig.from_hf_config(raw)).eval()
        weights = golden_weights(raw, SEEDS[name])
        state = model.state_dict()
        assert set(weights) == {k for k in state if not (raw["tie_word_embeddings"] and k == "lm_head.weight")}, \
            sorted(set(state) ^ set(weights))
        with torch.no_grad():
            for key, value in weights.items():
                state[key].copy_(value)
            prompt = golden_prompt(name)
            ids = torch.tensor([prompt])
            logits = model(input_ids=ids, use_cache=False).logits[0].float()
            if raw.get("use_sliding_window"):
                tokens = prompt[:GREEDY_PROMPT]
                for _ in range(GREEDY_NEW):
                    step = model(input_ids=torch.tensor([tokens]), use_cache=False).logits[0, -1]
                    tokens.append(int(step.argmax()))
                greedy = torch.tensor(tokens[GREEDY_PROMPT:])
            else:
                greedy = model.greedy_generate(ids[:, :GREEDY_PROMPT], max_new_tokens=GREEDY_NEW)[0, GREEDY_PROMPT:]
        np.savez_compressed(HERE / f"{name}.npz", prompt=np.array(prompt, dtype=np.int64),
                            logits=logits.numpy().astype(np.float32), greedy=greedy.numpy().astype(np.int64))
        print(name, tuple(logits.shape), greedy.tolist(), f"max |logit| {float(logits.abs().max()):.3f}")


if __name__ == "__main__":
    main()
