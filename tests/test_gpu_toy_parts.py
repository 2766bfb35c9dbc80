"""Parts the library has never seen, defined here and registered from outside: a feed-forward with
routing, another position encoding and another norm, put into a toy architecture whose two layers
differ in every part.  Nothing under the package changes for it; the toys are written with plain tensor
operations and exist only to show what the registries, the layer specification and the step function
carry.  They are no model of anyone's."""
import json
import tempfile

import pytest
import torch

import plain_qwen3 as plain
from gpu_util import assert_close
from qwen_triton_b200 import Engine, StepEntry, register_architecture
from qwen_triton_b200.config import LayerCall, LayerSpec, ModelSpec, PartSpec, config_from_dict
from qwen_triton_b200.engine.model import expected_tensors
from qwen_triton_b200.ops import kernels
from qwen_triton_b200.ops.kernels import GemmOut
from qwen_triton_b200.parts import register_feed_forward, register_norm, register_position
from qwen_triton_b200.weights import write_safetensors
from qwen_triton_b200.weights.tensors import TensorSpec

pytestmark = pytest.mark.gpu
DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16}


class ToyRoutedFeedForward:
    """Each token goes to the expert with the largest router logit (computed in float32) and gets
    silu(x G_e^T) * (x U_e^T) D_e^T scaled by that logit's sigmoid.  It gathers rows on the host's say, so it does
    not declare itself graph_safe: the engine must then run one-token steps without CUDA graphs."""

    def __init__(self, params, prefix, runtime):
        self.prefix, self.runtime = prefix, runtime
        self.hidden, self.inter, self.experts = int(params["hidden_size"]), int(params["intermediate_size"]), int(params["experts"])

    @classmethod
    def expected_tensors(cls, params, prefix):
        h, i, e = int(params["hidden_size"]), int(params["intermediate_size"]), int(params["experts"])
        return {f"{prefix}.router.weight": TensorSpec((e, h), role="vector", init_std=0.5),      # kept in 32-bit
                f"{prefix}.gate": TensorSpec((e, i, h), init_std=0.1),
                f"{prefix}.up": TensorSpec((e, i, h), init_std=0.1),
                f"{prefix}.down": TensorSpec((e, h, i), init_std=0.1)}

    def load(self, source):
        dev, dt = self.runtime.device, self.runtime.dtype
        self.router = source(f"{self.prefix}.router.weight").to(dev, torch.float32)
        self.gate, self.up, self.down = (source(f"{self.prefix}.{n}").to(dev, dt) for n in ("gate", "up", "down"))

    def forward(self, x, ctx):
        logits = x.float() @ self.router.T
        choice = logits.argmax(dim=-1)
        out = torch.zeros(x.shape[0], self.hidden, dtype=torch.float32, device=x.device)
        for e in range(self.experts):
            rows = (choice == e).nonzero().flatten()
            if rows.numel():
                xe = x[rows]
                act = (torch.nn.functional.silu((xe @ self.gate[e].T).float()) * (xe @ self.up[e].T).float()).to(x.dtype)
                out[rows] = (act @ self.down[e].T).float() * torch.sigmoid(logits[rows, e])[:, None]
        return GemmOut(out.to(self.runtime.dtype)[None].contiguous())


class ToySlowedRotary:
    """Rotary angles of position / slowdown: the table interface is all a position encoding needs."""

    def __init__(self, params, runtime):
        self.theta, self.rotary_dim, self.slowdown = float(params["theta"]), int(params["rotary_dim"]), float(params["slowdown"])
        self.runtime = runtime

    def key(self):
        return ("toy_slowed_rope", self.theta, self.rotary_dim, self.slowdown)

    def table(self, max_positions):
        cos, sin = plain.rope_tables(torch.arange(max_positions) / self.slowdown, self.rotary_dim, self.theta, torch.float32)
        return torch.cat((cos, sin), dim=-1).contiguous().to(self.runtime.device)


class ToyOffsetNorm:
    """x * rsqrt(mean(x^2) + eps) * (1 + w): the library's fused kernel with the weight shifted at load."""

    graph_safe = True           # launches one kernel and reads nothing back

    def __init__(self, params, name, runtime):
        self.size, self.eps, self.name, self.runtime = int(params["size"]), float(params["eps"]), name, runtime
        runtime.workspace.declare("toy_normed", runtime.max_step_tokens * self.size, runtime.dtype)

    @classmethod
    def expected_tensors(cls, params, name):
        return {f"{name}.offset": TensorSpec((int(params["size"]),), role="vector", init_std=0.1)}

    def load(self, source):
        self.weight = (1.0 + source(f"{self.name}.offset").float()).to(self.runtime.device).contiguous()

    def apply(self, stream, rows=None):
        count = stream.residual.shape[0] if rows is None else rows.shape[0]
        out = self.runtime.workspace.view("toy_normed", count, self.size)
        kernels.add_rmsnorm(stream.residual, stream.pending, self.weight, self.eps, out, rows)
        if rows is None:
            stream.pending = None
        return out


class ToyRoutedConfig:
    def __init__(self, raw):
        self.raw = dict(raw)

    @classmethod
    def from_hf_config(cls, raw):
        return cls(raw)

    def to_hf_dict(self):
        return dict(self.raw)

    def model_spec(self):
        r = self.raw
        hidden = r["hidden_size"]

        def attention(position, heads, kv_heads, head_dim, window):
            return PartSpec("attention", {"hidden_size": hidden, "num_heads": heads, "num_kv_heads": kv_heads, "head_dim": head_dim,
                                          "window": window, "qk_norm": True, "qk_norm_eps": r["eps"], "position": position,
                                          "q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj", "q_norm": "q_norm", "k_norm": "k_norm"})

        block = PartSpec("pre_norm", {"mixer": "attn", "feed_forward": "ff", "mixer_norm": "norm1", "feed_forward_norm": "norm2"})
        slowed = PartSpec("toy_slowed_rope", {"theta": r["theta"], "rotary_dim": 16, "slowdown": r["slowdown"]})
        plain_rope = PartSpec("rope", {"theta": r["theta"], "rotary_dim": 32, "head_dim": 32})
        layers = (
            LayerSpec("l0", block, attention(slowed, 4, 2, 16, None),
                      PartSpec("toy_routed", {"hidden_size": hidden, "intermediate_size": r["inter"], "experts": r["experts"]}),
                      PartSpec("toy_offset_norm", {"size": hidden, "eps": r["eps"]})),
            LayerSpec("l1", block, attention(plain_rope, 3, 1, 32, r["window"]),
                      PartSpec("gated_mlp", {"hidden_size": hidden, "intermediate_size": 2 * r["inter"], "activation": "silu"}),
                      PartSpec("rmsnorm", {"size": hidden, "eps": r["eps"]})),
        )
        return ModelSpec(architecture="ToyRoutedForCausalLM", vocab_size=r["vocab"], hidden_size=hidden,
                         embedding=PartSpec("token_embedding", {"name": "embed.weight"}), layers=layers,
                         schedule=(LayerCall(0), LayerCall(1)),
                         final_norm=PartSpec("toy_offset_norm", {"size": hidden, "eps": r["eps"], "name": "final"}),
                         head=PartSpec("linear_head", {"name": "head.weight"}), max_positions=256)


def oracle(raw, w, tokens):
    """The toy architecture in plain float32 over the whole sequence, one function per part."""
    eps, n = raw["eps"], len(tokens)
    x = w["embed.weight"][torch.tensor(tokens)]

    def offset_norm(h, name):
        return plain.rms_norm(h, 1.0 + w[f"{name}.offset"], eps)

    def attention(h, p, heads, kv_heads, d, cos, sin, window):
        q = plain.rms_norm((h @ w[f"{p}.q_proj.weight"].T).view(n, heads, d), w[f"{p}.q_norm.weight"], eps)
        k = plain.rms_norm((h @ w[f"{p}.k_proj.weight"].T).view(n, kv_heads, d), w[f"{p}.k_norm.weight"], eps)
        v = (h @ w[f"{p}.v_proj.weight"].T).view(n, kv_heads, d)
        q, k = plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin)
        return plain.attention_scores(q, k, v, d ** -0.5, window).reshape(n, heads * d) @ w[f"{p}.o_proj.weight"].T

    def routed(h, p):
        logits = h @ w[f"{p}.router.weight"].T
        choice = logits.argmax(-1)
        rows = []
        for t in range(n):
            e = int(choice[t])
            act = torch.nn.functional.silu(h[t] @ w[f"{p}.gate"][e].T) * (h[t] @ w[f"{p}.up"][e].T)
            rows.append((act @ w[f"{p}.down"][e].T) * torch.sigmoid(logits[t, e]))
        return torch.stack(rows), logits

    slow = plain.rope_tables(torch.arange(n) / raw["slowdown"], 16, raw["theta"], torch.float32)
    x = x + attention(offset_norm(x, "l0.norm1"), "l0.attn", 4, 2, 16, *slow, None)
    delta, router_logits = routed(offset_norm(x, "l0.norm2"), "l0.ff")
    x = x + delta
    fast = plain.rope_tables(torch.arange(n), 32, raw["theta"], torch.float32)
    x = x + attention(plain.rms_norm(x, w["l1.norm1.weight"], eps), "l1.attn", 3, 1, 32, *fast, raw["window"])
    x = x + plain.gated_mlp(plain.rms_norm(x, w["l1.norm2.weight"], eps),
                            {k.replace("l1.ff.", "m.", 1): v for k, v in w.items() if k.startswith("l1.ff.")}, "m")
    return offset_norm(x, "final") @ w["head.weight"].T, router_logits


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_toy_routed_feed_forward_position_and_norm_register_build_and_step(dtype):
    register_feed_forward("toy_routed", ToyRoutedFeedForward)
    register_position("toy_slowed_rope", ToySlowedRotary)
    register_norm("toy_offset_norm", ToyOffsetNorm)
    register_architecture("ToyRoutedForCausalLM", ToyRoutedConfig)
    raw = {"architectures": ["ToyRoutedForCausalLM"], "hidden_size": 48, "inter": 40, "experts": 3, "vocab": 83, "eps": 3e-6,
           "theta": 5e3, "slowdown": 4.0, "window": 6}
    config = config_from_dict(raw)
    assert isinstance(config, ToyRoutedConfig)
    expected = expected_tensors(config.model_spec())
    assert {"l0.ff.router.weight", "l0.norm1.offset", "l1.norm1.weight", "final.offset", "head.weight"} <= set(expected)
    weights = {}
    for index, (name, spec) in enumerate(sorted(expected.items())):
        g = torch.Generator().manual_seed(400 + index)
        values = torch.randn(spec.shape, generator=g) * spec.init_std + spec.init_mean
        weights[name] = values.float() if spec.role == "vector" else values.to(DTYPES[dtype])
    with tempfile.TemporaryDirectory() as folder:
        write_safetensors(f"{folder}/model.safetensors", weights)
        with open(f"{folder}/config.json", "w") as handle:
            json.dump(raw, handle)
        engine = Engine.from_pretrained(folder, dtype=dtype, max_tokens=512)
    assert len(engine.cache.groups) == 2                       # all keys for layer 0, a window of them for layer 1
    wf = {k: v.float() for k, v in weights.items()}
    requests = [[5, 9, 2, 77, 30, 11, 4, 8, 60, 1, 13, 44, 7], [35, 53, 16]]      # chosen for wide routing margins
    for i, tokens in enumerate(requests):
        want, router_logits = oracle(raw, wf, tokens)
        top2 = router_logits.topk(2, dim=-1).values
        assert float((top2[:, 0] - top2[:, 1]).min()) > 0.05, "the test wants routing decisions that rounding cannot flip"
        assert i or router_logits.argmax(-1).unique().numel() > 1, "the longer request should reach more than one expert"
        slot = engine.new_sequence()
        whole = engine.step([StepEntry(slot, tokens, list(range(len(tokens))))])
        engine.release(slot)
        assert_close(whole, want, dtype, f"toy routed model, request {i} whole")
    # prompts of unequal length in one step, then one token each until the shorter request ends
    slots = [engine.new_sequence() for _ in requests]
    rows = {0: [], 1: []}
    first = engine.step([StepEntry(slots[0], requests[0][:5], [0, 1, 2, 3, 4]), StepEntry(slots[1], requests[1][:2], [0, 1])])
    rows[0].append(first[:5])
    rows[1].append(first[5:])
    at = [5, 2]
    while any(a < len(r) for a, r in zip(at, requests)):
        live = [i for i in (0, 1) if at[i] < len(requests[i])]
        out = engine.step([StepEntry(slots[i], [requests[i][at[i]]], [0]) for i in live])
        for row, i in enumerate(live):
            rows[i].append(out[row:row + 1])
            at[i] += 1
    for i in (0, 1):
        assert_close(torch.cat(rows[i]), oracle(raw, wf, requests[i])[0], dtype, f"toy routed model, request {i} step by step")
        engine.release(slots[i])
    assert engine.graph_replays == 0                           # a part that is not graph_safe keeps the whole model out of graphs
