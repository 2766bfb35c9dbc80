"""Plain, slow implementation of the Qwen3 dense architecture: the tests' oracle.

Written from the formulas of luozoupi/Qwen-Triton (each function cites the
file and lines it restates).  Whole sequences only, no cache, one function per
part, float32 (or float64 on request) throughout, plain tensor operations, on whatever device
its weights lie (a large model's oracle runs on the GPU, with library products in full precision).  It
shares no code with the ``qwen_triton_b200`` package: it reads the raw
config.json mapping itself and takes weights as a ``name -> tensor`` mapping.

``tests/golden/`` holds logits that the reference's own model code produced on
the CPU for tiny random models; ``tests/test_plain_vs_golden.py`` checks this
file against them.
"""
from __future__ import annotations

import math
from typing import Mapping, Sequence

import torch


# ----------------------------------------------------------------------------- config
def read_config(raw: Mapping) -> dict:
    """The few keys the formulas need, with the reference's defaults
    (qwen_triton/configs/config.py:120-176)."""
    text = dict(raw.get("text_config") or raw)
    layers = int(text["num_hidden_layers"])
    heads = int(text["num_attention_heads"])
    hidden = int(text["hidden_size"])
    head_dim = int(text.get("head_dim") or hidden // heads)                      # config.py:139
    rope_params = dict(text.get("rope_parameters") or {})
    theta = float(text.get("rope_theta") or rope_params.get("rope_theta") or 10000.0)   # config.py:140-144
    partial = float(text.get("partial_rotary_factor") or rope_params.get("partial_rotary_factor") or 1.0)
    rotary_dim = max(2, int(head_dim * partial))                                 # config.py:103-109
    rotary_dim -= rotary_dim % 2
    use_window = bool(text.get("use_sliding_window", False))
    window = text.get("sliding_window")
    layer_types = text.get("layer_types")
    if not layer_types:                                                          # config.py:22-28
        if use_window and window is not None:
            cutoff = text.get("max_window_layers")
            cutoff = layers if cutoff is None else int(cutoff)
            layer_types = ["sliding_attention" if i >= cutoff else "full_attention" for i in range(layers)]
        else:
            layer_types = ["full_attention"] * layers
    return {
        "layers": layers, "heads": heads, "kv_heads": int(text.get("num_key_value_heads") or heads),
        "hidden": hidden, "head_dim": head_dim, "intermediate": int(text["intermediate_size"]),
        "vocab": int(text["vocab_size"]), "eps": float(text.get("rms_norm_eps", 1e-6)),
        "theta": theta, "rotary_dim": rotary_dim,
        "tied": bool(raw.get("tie_word_embeddings", text.get("tie_word_embeddings", False))),   # config.py:165
        "window": int(window) if window is not None else None, "layer_types": list(layer_types),
        "attention_bias": bool(text.get("attention_bias", False)),              # config.py:150-151
    }


# ----------------------------------------------------------------------------- parts
def _wide(x: torch.Tensor) -> torch.Tensor:
    """float32 and float64 stay; a 16-bit model dtype is widened to float32, as the reference's kernels do inside
    norms, rotation, softmax and the SiLU gate before they round their result once to the model dtype."""
    return x if x.dtype in (torch.float32, torch.float64) else x.float()


def embed(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """Row gather (qwen_triton/kernels/embedding.py:34-35)."""
    return table[ids]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w over the last dim (qwen_triton/kernels/rmsnorm.py:35-42)."""
    wide = _wide(x)
    variance = wide.pow(2).mean(dim=-1, keepdim=True)
    return (wide * torch.rsqrt(variance + eps) * _wide(weight)).to(x.dtype)


def rope_tables(positions: torch.Tensor, rotary_dim: int, theta: float, dtype: torch.dtype):
    """inv_freq[j] = theta^(-2j/rd); angle = pos * inv_freq; cos/sin of the angle
    (qwen_triton/modules/rotary.py:14-26).  Returns the half tables [S, rd/2]."""
    exponent = torch.arange(0, rotary_dim, 2, dtype=torch.float32, device=positions.device) / rotary_dim
    work = dtype if dtype in (torch.float32, torch.float64) else torch.float32      # rotary.py:22: angles in float32
    inv_freq = (1.0 / (theta ** exponent)).to(work)
    angles = positions.to(work)[:, None] * inv_freq[None, :]
    return angles.cos().to(dtype), angles.sin().to(dtype)                           # rotary.py:25-26: tables in the model dtype


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half on x [S, heads, d]: o1 = x1 cos - x2 sin, o2 = x2 cos + x1 sin; dims beyond
    the rotary width pass through (qwen_triton/kernels/rope.py:59-69)."""
    half = cos.shape[-1]
    wide = _wide(x)
    x1, x2, rest = wide[..., :half], wide[..., half:2 * half], wide[..., 2 * half:]
    c, s = _wide(cos)[:, None, :], _wide(sin)[:, None, :]
    return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s, rest), dim=-1).to(x.dtype)


def attention_scores(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                     window: int | None) -> torch.Tensor:
    """Causal softmax attention of one sequence that starts at position 0.

    q [S, nq, d], k/v [S, nkv, d].  Query head h uses kv head h // (nq/nkv)
    (qwen_triton/modules/attention.py:17-22,33).  Key j is visible to the query at position p
    iff j <= p, and j > p - window for a windowed layer (qwen_triton/models/core.py:58-61);
    hidden scores are set to the most negative float before the softmax (core.py:63-65);
    scores are scaled by ``scale`` (attention.py:34,122).
    """
    seq, nq, d = q.shape
    groups = nq // k.shape[1]
    out_dtype = q.dtype
    q, k, v = _wide(q), _wide(k), _wide(v)                       # attention.py:110-123: scores, softmax and PV in float32
    k = k.repeat_interleave(groups, dim=1)
    v = v.repeat_interleave(groups, dim=1)
    scores = torch.einsum("qhd,khd->hqk", q, k) * scale
    pos = torch.arange(seq, device=q.device)
    visible = pos[None, :] <= pos[:, None]
    if window is not None:
        visible &= pos[None, :] > (pos[:, None] - window)
    scores = scores.masked_fill(~visible[None], torch.finfo(scores.dtype).min)
    probs = torch.softmax(scores, dim=-1)
    return torch.einsum("hqk,khd->qhd", probs, v).to(out_dtype)


def attention_layer(x: torch.Tensor, w: Mapping[str, torch.Tensor], prefix: str, cfg: dict,
                    window: int | None) -> torch.Tensor:
    """q/k/v projections, per-head q_norm/k_norm before RoPE, attention, output projection
    (qwen_triton/modules/attention.py:53-73,125-128); with ``attention_bias`` all four projections have a bias
    (attention.py:38-41), added to the product after it was rounded (modules/linear.py:31, kernels/matmul.py:99-111)."""
    seq = x.shape[0]
    d = cfg["head_dim"]

    def project(name: str, rows: torch.Tensor) -> torch.Tensor:
        out = rows @ w[f"{prefix}.{name}.weight"].T
        return out + w[f"{prefix}.{name}.bias"] if cfg.get("attention_bias", False) else out

    q = project("q_proj", x).view(seq, cfg["heads"], d)
    k = project("k_proj", x).view(seq, cfg["kv_heads"], d)
    v = project("v_proj", x).view(seq, cfg["kv_heads"], d)
    q = rms_norm(q, w[f"{prefix}.q_norm.weight"], cfg["eps"])
    k = rms_norm(k, w[f"{prefix}.k_norm.weight"], cfg["eps"])
    cos, sin = rope_tables(torch.arange(seq, device=x.device), cfg["rotary_dim"], cfg["theta"], x.dtype)
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    out = attention_scores(q, k, v, d ** -0.5, window)
    return project("o_proj", out.reshape(seq, cfg["heads"] * d))


def gated_mlp(x: torch.Tensor, w: Mapping[str, torch.Tensor], prefix: str) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)) (qwen_triton/modules/mlp.py:19-22; kernels/swiglu.py:35-36)."""
    gate = x @ w[f"{prefix}.gate_proj.weight"].T
    up = x @ w[f"{prefix}.up_proj.weight"].T
    act = (_wide(gate) * torch.sigmoid(_wide(gate)) * _wide(up)).to(x.dtype)        # swiglu.py:84-92: float32 inside, one rounding
    return act @ w[f"{prefix}.down_proj.weight"].T


def decoder_layer(x: torch.Tensor, w: Mapping[str, torch.Tensor], index: int, cfg: dict) -> torch.Tensor:
    """Pre-norm residual block (qwen_triton/models/core.py:126-152)."""
    prefix = f"model.layers.{index}"
    window = cfg["window"] if cfg["layer_types"][index] == "sliding_attention" else None
    h = rms_norm(x, w[f"{prefix}.input_layernorm.weight"], cfg["eps"])
    x = x + attention_layer(h, w, f"{prefix}.self_attn", cfg, window)
    h = rms_norm(x, w[f"{prefix}.post_attention_layernorm.weight"], cfg["eps"])
    return x + gated_mlp(h, w, f"{prefix}.mlp")


# ----------------------------------------------------------------------------- model
def prepare_weights(weights: Mapping[str, torch.Tensor], dtype: torch.dtype = torch.float32) -> dict:
    return {name: tensor.to(dtype) for name, tensor in weights.items()}


def forward(raw_config: Mapping, weights: Mapping[str, torch.Tensor], token_ids: Sequence[int],
            dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Logits [S, vocab] of one whole sequence (qwen_triton/models/core.py:181,230-242,364)."""
    cfg = read_config(raw_config)
    w = weights if all(t.dtype == dtype for t in weights.values()) else prepare_weights(weights, dtype)
    ids = torch.as_tensor(list(token_ids), dtype=torch.long)
    x = embed(ids, w["model.embed_tokens.weight"])
    for index in range(cfg["layers"]):
        x = decoder_layer(x, w, index, cfg)
    x = rms_norm(x, w["model.norm.weight"], cfg["eps"])
    head = w["model.embed_tokens.weight"] if cfg["tied"] else w["lm_head.weight"]     # core.py:262-263
    return x @ head.T


def greedy_generate(raw_config: Mapping, weights: Mapping[str, torch.Tensor], prompt: Sequence[int],
                    max_new_tokens: int, stop_ids: Sequence[int] = ()) -> list[int]:
    """argmax of the last position, append, repeat with the whole sequence
    (qwen_triton/models/core.py:392-409).  The reference has no stop condition; ``stop_ids`` ends the
    sequence after emitting the stop token."""
    w = prepare_weights(weights)
    tokens = list(prompt)
    new: list[int] = []
    for _ in range(max_new_tokens):
        logits = forward(raw_config, w, tokens)
        token = int(torch.argmax(logits[-1]))
        new.append(token)
        tokens.append(token)
        if token in stop_ids:
            break
    return new


# ----------------------------------------------------------------------------- sampling (not in the reference)
_MASK64 = (1 << 64) - 1


def _mix64(value: int) -> int:
    """The splitmix64 finaliser."""
    value = (value + 0x9E3779B97F4A7C15) & _MASK64
    value = ((value ^ (value >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    value = ((value ^ (value >> 27)) * 0x94D049BB133111EB) & _MASK64
    return value ^ (value >> 31)


def uniform_for(seed: int, request: int, step: int) -> float:
    """The uniform number in [0, 1) that request ``request`` uses for its ``step``-th new token:
    three rounds of splitmix64 over (seed, request, step), top 24 bits."""
    state = _mix64(seed & _MASK64)
    state = _mix64(state ^ (request & _MASK64))
    state = _mix64(state ^ (step & _MASK64))
    return (state >> 40) / float(1 << 24)


def sample_temperature(logits: torch.Tensor, temperature: float, uniform: float) -> int:
    """Inverse-CDF sample of softmax(logits / T) in vocabulary order: the first token whose
    cumulative weight exceeds ``uniform`` times the total weight."""
    scaled = logits.double() / temperature
    weights = torch.exp(scaled - scaled.max())
    cumulative = torch.cumsum(weights, dim=0)
    target = uniform * float(cumulative[-1])
    index = int(torch.searchsorted(cumulative, torch.tensor(target, dtype=torch.float64), right=True))
    return min(index, logits.numel() - 1)


def kept_tokens(logits: torch.Tensor, temperature: float, top_k: int = 0, top_p: float = 1.0) -> torch.Tensor:
    """Which tokens top_k and top_p leave to draw from (bool [vocab]), stated with a sort: the k largest logits and
    every logit equal to the k-th; then, with probabilities renormalised over those, the shortest run of the most
    likely tokens that sums to top_p and every token as likely as its last."""
    keep = torch.ones_like(logits, dtype=torch.bool)
    if 0 < top_k < logits.numel():
        keep &= logits >= torch.topk(logits, top_k).values[-1]
    if top_p < 1.0:
        scaled = logits.double() / temperature
        weights = torch.where(keep, torch.exp(scaled - scaled.max()), torch.zeros_like(scaled))
        ordered, order = torch.sort(weights, descending=True)
        reached = int(torch.searchsorted(torch.cumsum(ordered, dim=0), top_p * weights.sum()))
        keep &= logits >= logits[order[min(reached, logits.numel() - 1)]]
    return keep


def choice_is_consistent(logits: torch.Tensor, temperature: float, uniform: float, token: int,
                         slack: float = 1e-4, top_k: int = 0, top_p: float = 1.0) -> bool:
    """Whether ``token`` is the inverse-CDF choice for ``uniform`` up to float32 rounding of the
    cumulative weights: the target mass lies in the token's interval widened by ``slack`` of the total.  With
    ``top_k`` / ``top_p`` only the tokens of ``kept_tokens`` have weight."""
    scaled = logits.double() / temperature
    weights = torch.exp(scaled - scaled.max())
    if top_k or top_p < 1.0:
        keep = kept_tokens(logits, temperature, top_k, top_p)
        if not bool(keep[token]):
            return False
        weights = torch.where(keep, weights, torch.zeros_like(weights))
    cumulative = torch.cumsum(weights, dim=0)
    total = float(cumulative[-1])
    target = uniform * total
    lower = float(cumulative[token - 1]) if token > 0 else 0.0
    return lower - slack * total <= target <= float(cumulative[token]) + slack * total
