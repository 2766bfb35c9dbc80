"""Each part alone against the plain implementation's function for it, and a toy mixer with state of
its own that is registered, built and stepped without touching the library's files."""
import tempfile

import pytest
import torch

import plain_qwen3 as plain
from gpu_util import TOL, assert_close
from qwen_triton_b200 import Engine, StepEntry, register_architecture
from qwen_triton_b200.cache import SequenceCache
from qwen_triton_b200.config import LayerCall, LayerSpec, ModelSpec, PartSpec
from qwen_triton_b200.engine.step import StepContext
from qwen_triton_b200.ops.kernels import GemmOut
from qwen_triton_b200.parts import (ResidualStream, Runtime, StateRequest, Workspace, part_class, register_mixer)
from qwen_triton_b200.weights import write_safetensors
from qwen_triton_b200.weights.tensors import TensorSpec

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16}


def runtime(dtype, max_tokens=256, max_positions=512):
    return Runtime(device=DEV, dtype=DTYPES[dtype], max_step_tokens=max_tokens, max_positions=max_positions,
                   workspace=Workspace(DEV))


def weights_for(expected, dtype, seed=0):
    out = {}
    for index, (name, spec) in enumerate(sorted(expected.items())):
        g = torch.Generator().manual_seed(seed * 100 + index)
        values = torch.randn(spec.shape, generator=g) * (0.2 if spec.role == "vector" else 0.08) + spec.init_mean
        out[name] = values.to(DTYPES[dtype])
    return out


def context(rt, cache, lengths, past=None):
    past = past or [0] * len(lengths)
    slots = [cache.alloc() for _ in lengths]
    for slot, n, p in zip(slots, lengths, past):
        cache.book.extend(slot, p + n)
    import numpy as np
    tables = []
    for g in range(len(cache.groups)):
        width = max(len(cache.book.pages(s, g)) for s in slots)
        table = np.zeros((len(slots), width), dtype=np.int32)
        for i, s in enumerate(slots):
            table[i, :len(cache.book.pages(s, g))] = cache.book.pages(s, g)
        tables.append(table)
    meta = torch.zeros(StepContext.meta_size(sum(lengths), len(lengths), [t.shape[1] for t in tables]), dtype=torch.int32, device=DEV)
    ctx = StepContext(device=DEV, meta=meta)
    ctx.fill(slots, [[0] * n for n in lengths], past, [], tables)
    return ctx, slots


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_norm_part(dtype):
    rt = runtime(dtype)
    norm = part_class("norm", PartSpec("rmsnorm"))({"size": 200, "eps": 2e-5}, "n", rt)
    expected = norm.expected_tensors({"size": 200, "eps": 2e-5}, "n")
    assert list(expected) == ["n.weight"] and expected["n.weight"].role == "vector"
    w = weights_for(expected, dtype)
    norm.load(w.__getitem__)
    rt.workspace.allocate()
    x = torch.randn(9, 200, generator=torch.Generator().manual_seed(1))
    delta = (torch.randn(9, 200, generator=torch.Generator().manual_seed(2))).to(DTYPES[dtype])
    stream = ResidualStream(x.to(DEV).clone())
    stream.add(GemmOut(delta.to(DEV)[None]))
    out = norm.apply(stream)
    assert stream.pending is None
    want = plain.rms_norm(x + delta.float(), w["n.weight"].float(), 2e-5)
    assert_close(out, want, dtype, "norm part")
    assert norm.weight.dtype == torch.float32                    # vectors are kept in 32-bit


def test_position_part_matches_the_formula():
    rt = runtime("fp32")
    rope = part_class("position", PartSpec("rope"))({"theta": 1e6, "rotary_dim": 24, "head_dim": 32}, rt)
    table = rope.table(300).cpu()
    cos, sin = plain.rope_tables(torch.arange(300), 24, 1e6, torch.float32)
    assert table.dtype == torch.float32 and torch.equal(table, torch.cat((cos, sin), -1))
    assert part_class("position", PartSpec("none"))({}, rt).table(10) is None
    with pytest.raises(ValueError):
        part_class("position", PartSpec("rope"))({"theta": 1e4, "rotary_dim": 34, "head_dim": 32}, rt)


ATTN = {"hidden_size": 72, "num_heads": 6, "num_kv_heads": 2, "head_dim": 48, "qk_norm": True, "qk_norm_eps": 1e-5,
        "position": PartSpec("rope", {"theta": 7e4, "rotary_dim": 48, "head_dim": 48}),
        "q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj", "q_norm": "q_norm", "k_norm": "k_norm"}


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("window", [None, 10])
def test_attention_part(dtype, window):
    rt = runtime(dtype)
    params = {**ATTN, "window": window}
    mixer = part_class("mixer", PartSpec("attention"))(params, "a", rt)
    w = weights_for(mixer.expected_tensors(params, "a"), dtype, seed=3)
    mixer.load(w.__getitem__)
    rt.workspace.allocate()
    cache = SequenceCache([mixer.cache_request()], [None], max_tokens=512, max_seq_len=512, dtype=DTYPES[dtype], device=DEV,
                          chunk_tokens=64)
    lengths = [40, 7]
    ctx, _ = context(rt, cache, lengths)
    x = (torch.randn(sum(lengths), 72, generator=torch.Generator().manual_seed(4)) * 0.5).to(DTYPES[dtype])
    out = mixer.forward(x.to(DEV), ctx, cache.view(0)).value()
    cfg = {"heads": 6, "kv_heads": 2, "head_dim": 48, "eps": 1e-5, "rotary_dim": 48, "theta": 7e4}
    wf = {k: v.float() for k, v in w.items()}
    start = 0
    for n in lengths:
        want = plain.attention_layer(x[start:start + n].float(), wf, "a", cfg, window)
        assert_close(out[start:start + n], want, dtype, f"attention part, window={window}")
        start += n


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("head_dim, lengths", [(48, [40, 7]), (32, [9, 4]), (32, [200, 90])])
def test_attention_part_with_neighbours_as_rotation_pairs(dtype, head_dim, lengths):
    """``pairing: interleaved`` on the position part: elements (2i, 2i + 1) of a head turn together.  Head size 32 with
    13 tokens takes the fused projection (in bfloat16), the other cases the separate kernel."""
    from test_gpu_kernels import rope_interleaved
    rt = runtime(dtype, max_tokens=512)
    position = PartSpec("rope", {"theta": 7e4, "rotary_dim": head_dim, "head_dim": head_dim, "pairing": "interleaved"})
    params = {**ATTN, "head_dim": head_dim, "position": position, "window": None}
    mixer = part_class("mixer", PartSpec("attention"))(params, "a", rt)
    assert mixer.interleaved
    w = weights_for(mixer.expected_tensors(params, "a"), dtype, seed=13)
    mixer.load(w.__getitem__)
    rt.workspace.allocate()
    cache = SequenceCache([mixer.cache_request()], [None], max_tokens=1024, max_seq_len=512, dtype=DTYPES[dtype], device=DEV)
    ctx, _ = context(rt, cache, lengths)
    x = (torch.randn(sum(lengths), 72, generator=torch.Generator().manual_seed(4)) * 0.5).to(DTYPES[dtype])
    out = mixer.forward(x.to(DEV), ctx, cache.view(0)).value()
    wf = {k: v.float() for k, v in w.items()}
    nq, nkv, start = ATTN["num_heads"], ATTN["num_kv_heads"], 0
    for n in lengths:
        h = x[start:start + n].float()
        q = plain.rms_norm((h @ wf["a.q_proj.weight"].T).view(n, nq, head_dim), wf["a.q_norm.weight"], 1e-5)
        k = plain.rms_norm((h @ wf["a.k_proj.weight"].T).view(n, nkv, head_dim), wf["a.k_norm.weight"], 1e-5)
        v = (h @ wf["a.v_proj.weight"].T).view(n, nkv, head_dim)
        cos, sin = plain.rope_tables(torch.arange(n), head_dim, 7e4, torch.float32)
        q, k = rope_interleaved(q, cos, sin), rope_interleaved(k, cos, sin)
        want = plain.attention_scores(q, k, v, head_dim ** -0.5, None).reshape(n, nq * head_dim) @ wf["a.o_proj.weight"].T
        assert_close(out[start:start + n], want, dtype, "attention part, neighbours as pairs")
        start += n


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("inter, tokens", [(200, 11), (208, 11), (208, 300)])    # 208: gate and up interleaved in bfloat16; 300 tokens: gated in the GEMM
def test_feed_forward_part(dtype, inter, tokens):
    rt = runtime(dtype, max_tokens=512)
    params = {"hidden_size": 72, "intermediate_size": inter, "activation": "silu", "gate": "gate_proj", "up": "up_proj", "down": "down_proj"}
    ff = part_class("feed_forward", PartSpec("gated_mlp"))(params, "m", rt)
    w = weights_for(ff.expected_tensors(params, "m"), dtype, seed=5)
    ff.load(w.__getitem__)
    rt.workspace.allocate()
    x = (torch.randn(tokens, 72, generator=torch.Generator().manual_seed(6))).to(DTYPES[dtype])
    out = ff.forward(x.to(DEV), None).value()
    assert_close(out, plain.gated_mlp(x.float(), {k: v.float() for k, v in w.items()}, "m"), dtype, "feed-forward part")
    with pytest.raises(ValueError, match="activation"):
        part_class("feed_forward", PartSpec("gated_mlp"))({**params, "activation": "softplus"}, "m", rt)


@pytest.mark.parametrize("tokens", [9, 300])
def test_feed_forward_part_with_another_activation(tokens):
    """The gate's activation is a parameter of the part: GELU here, through the few-token and the many-token kernels."""
    rt = runtime("bf16", max_tokens=512)
    params = {"hidden_size": 72, "intermediate_size": 208, "activation": "gelu_pytorch_tanh"}
    ff = part_class("feed_forward", PartSpec("gated_mlp"))(params, "m", rt)
    w = weights_for(ff.expected_tensors(params, "m"), "bf16", seed=5)
    ff.load(w.__getitem__)
    rt.workspace.allocate()
    x = torch.randn(tokens, 72, generator=torch.Generator().manual_seed(6)).to(torch.bfloat16)
    wf = {k: v.float() for k, v in w.items()}
    gate, up = x.float() @ wf["m.gate_proj.weight"].T, x.float() @ wf["m.up_proj.weight"].T
    want = (torch.nn.functional.gelu(gate, approximate="tanh") * up).to(torch.bfloat16).float() @ wf["m.down_proj.weight"].T
    assert_close(ff.forward(x.to(DEV), None).value(), want, "bf16", "feed-forward part with GELU")


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_block_part(dtype):
    rt = runtime(dtype)
    layer = LayerSpec(prefix="model.layers.0",
                      block=PartSpec("pre_norm", {"mixer": "self_attn", "feed_forward": "mlp", "mixer_norm": "input_layernorm",
                                                  "feed_forward_norm": "post_attention_layernorm"}),
                      mixer=PartSpec("attention", {**ATTN, "window": None}),
                      feed_forward=PartSpec("gated_mlp", {"hidden_size": 72, "intermediate_size": 136, "activation": "silu"}),
                      norm=PartSpec("rmsnorm", {"size": 72, "eps": 1e-5}))
    block = part_class("block", layer.block)(layer, rt)
    w = weights_for(block.expected_tensors(layer), dtype, seed=7)
    assert len(w) == 11
    block.load(w.__getitem__)
    rt.workspace.declare("residual", 256 * 72, torch.float32)
    rt.workspace.allocate()
    cache = SequenceCache([block.mixer.cache_request()], [None], max_tokens=512, max_seq_len=512, dtype=DTYPES[dtype], device=DEV)
    ctx, _ = context(rt, cache, [23])
    x = torch.randn(23, 72, generator=torch.Generator().manual_seed(8)).to(DTYPES[dtype]).float()
    stream = ResidualStream(x.to(DEV).clone())
    block.forward(stream, ctx, cache.view(0))
    got = stream.residual + stream.pending.value()
    cfg = {"heads": 6, "kv_heads": 2, "head_dim": 48, "eps": 1e-5, "rotary_dim": 48, "theta": 7e4, "window": None,
           "layer_types": ["full_attention"]}
    want = plain.decoder_layer(x, {k: v.float() for k, v in w.items()}, 0, cfg)
    assert_close(got, want, dtype, "block part")


# ----------------------------------------------------------------------------- a toy mixer with state of its own
class ToyDecayMixer:
    """s_t = decay * s_{t-1} + x_t W per sequence, output s_t: a recurrent mixer whose only memory is a
    fixed-size state block per sequence.  Written with plain tensor operations; it exists to show that
    the library's registries, cache and step function carry a mixer they have never seen."""

    def __init__(self, params, prefix, runtime):
        self.prefix, self.runtime = prefix, runtime
        self.hidden, self.decay = int(params["hidden_size"]), float(params["decay"])
        self.weight = None

    @classmethod
    def expected_tensors(cls, params, prefix):
        return {f"{prefix}.mix.weight": TensorSpec((int(params["hidden_size"]),) * 2, init_std=0.1)}

    def load(self, source):
        self.weight = source(f"{self.prefix}.mix.weight").to(self.runtime.device, torch.float32)

    def cache_request(self):
        return StateRequest((self.hidden,), torch.float32)

    def forward(self, x, ctx, cache):
        projected = x.float() @ self.weight.T
        out = torch.empty_like(projected)
        starts, slots = ctx.seq_start.tolist(), ctx.slots.tolist()
        for b, slot in enumerate(slots):
            state = cache.state[slot]
            for t in range(starts[b], starts[b + 1]):
                state = self.decay * state + projected[t]
                out[t] = state
            cache.state[slot] = state
        return GemmOut(out.to(self.runtime.dtype)[None].contiguous())


class ToyConfig:
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
        norm = PartSpec("rmsnorm", {"size": hidden, "eps": r["eps"]})
        block = PartSpec("pre_norm", {"mixer": "mixer", "feed_forward": "ff", "mixer_norm": "norm1", "feed_forward_norm": "norm2"})
        ff = PartSpec("gated_mlp", {"hidden_size": hidden, "intermediate_size": r["inter"], "activation": "silu"})
        toy = PartSpec(r.get("mixer_kind", "toy_decay"), {"hidden_size": hidden, "decay": r["decay"]})
        attn = PartSpec("attention", {"hidden_size": hidden, "num_heads": 2, "num_kv_heads": 1, "head_dim": 16, "window": None,
                                      "qk_norm": False, "position": PartSpec("none"),
                                      "q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj"})
        layers = (LayerSpec("blocks.0", block, toy, ff, norm), LayerSpec("blocks.1", block, attn, ff, norm))
        # layer 0 runs twice (two state entries), and the last call reads the keys the attention call before it wrote
        schedule = (LayerCall(0), LayerCall(1), LayerCall(0), LayerCall(1, cache_of=1))
        return ModelSpec(architecture="ToyForCausalLM", vocab_size=r["vocab"], hidden_size=hidden,
                         embedding=PartSpec("token_embedding", {"name": "embed.weight"}), layers=layers, schedule=schedule,
                         final_norm=PartSpec("rmsnorm", {"size": hidden, "eps": r["eps"], "name": "final"}),
                         head=PartSpec("linear_head", {"name": "head.weight", "tied_to": "embed.weight"}), max_positions=256)


def toy_oracle(raw, w, tokens):
    """The toy model in plain float32, whole sequence."""
    hidden, eps = raw["hidden_size"], raw["eps"]
    x = w["embed.weight"][torch.tensor(tokens)]
    n = len(tokens)

    def ff(h, p):
        return plain.gated_mlp(h, {k.replace(f"{p}.ff.", "m.", 1): v for k, v in w.items() if k.startswith(f"{p}.ff.")}, "m")

    def toy(h, p):
        proj = h @ w[f"{p}.mixer.mix.weight"].T
        state, out = torch.zeros(hidden), []
        for t in range(n):
            state = raw["decay"] * state + proj[t]
            out.append(state)
        return torch.stack(out)

    def attn(h, p):
        q = (h @ w[f"{p}.mixer.q_proj.weight"].T).view(n, 2, 16)
        k = (h @ w[f"{p}.mixer.k_proj.weight"].T).view(n, 1, 16)
        v = (h @ w[f"{p}.mixer.v_proj.weight"].T).view(n, 1, 16)
        return plain.attention_scores(q, k, v, 16 ** -0.5, None).reshape(n, 32) @ w[f"{p}.mixer.o_proj.weight"].T, k, v

    kept = None
    for position, (layer, mix) in enumerate([("blocks.0", "toy"), ("blocks.1", "attn"), ("blocks.0", "toy"), ("blocks.1", "shared")]):
        h = plain.rms_norm(x, w[f"{layer}.norm1.weight"], eps)
        if mix == "toy":
            x = x + toy(h, layer)
        elif mix == "attn":
            delta, k, v = attn(h, layer)
            kept = (k, v)
            x = x + delta
        else:                                                  # queries of this call over the keys and values of the earlier call
            q = (h @ w[f"{layer}.mixer.q_proj.weight"].T).view(n, 2, 16)
            x = x + plain.attention_scores(q, kept[0], kept[1], 16 ** -0.5, None).reshape(n, 32) @ w[f"{layer}.mixer.o_proj.weight"].T
        x = x + ff(plain.rms_norm(x, w[f"{layer}.norm2.weight"], eps), layer)
    return plain.rms_norm(x, w["final.weight"], eps) @ w["embed.weight"].T


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_toy_mixer_with_state_registers_builds_and_steps(dtype):
    register_mixer("toy_decay", ToyDecayMixer)
    register_architecture("ToyForCausalLM", ToyConfig)
    raw = {"architectures": ["ToyForCausalLM"], "hidden_size": 40, "inter": 56, "vocab": 97, "eps": 1e-5, "decay": 0.8}
    from qwen_triton_b200.config import config_from_dict
    from qwen_triton_b200.engine.model import expected_tensors
    config = config_from_dict(raw)
    assert isinstance(config, ToyConfig)
    expected = expected_tensors(config.model_spec())
    weights = weights_for(expected, dtype, seed=9)
    with tempfile.TemporaryDirectory() as folder:
        write_safetensors(f"{folder}/model.safetensors", weights)
        import json
        with open(f"{folder}/config.json", "w") as handle:
            json.dump(raw, handle)
        engine = Engine.from_pretrained(folder, dtype=dtype, max_tokens=512)
    assert len(engine.cache.groups) == 1 and len(engine.cache.groups[0].owners) == 1      # one attention entry, shared by two calls
    assert engine.cache.view(0).state is not engine.cache.view(2).state                   # the layer that runs twice has two states
    wf = {k: v.float() for k, v in weights.items()}
    requests = [[5, 9, 2, 77, 30, 11, 4, 8, 60, 1, 13], [96, 0, 41]]
    whole = {}
    for i, tokens in enumerate(requests):
        slot = engine.new_sequence()
        whole[i] = engine.step([StepEntry(slot, tokens, list(range(len(tokens))))])
        engine.release(slot)
        assert_close(whole[i], toy_oracle(raw, wf, tokens), dtype, f"toy model, request {i} whole")
    # both requests as a batch: prompts of unequal length, then one token each; slots are the ones just given back,
    # so their state must have been cleared
    slots = [engine.new_sequence() for _ in requests]
    rows = {0: [], 1: []}
    first = engine.step([StepEntry(slots[0], requests[0][:4], [0, 1, 2, 3]), StepEntry(slots[1], requests[1][:1], [0])])
    rows[0].append(first[:4])
    rows[1].append(first[4:])
    for t in range(7):
        entries, owners = [], []
        for i in (0, 1):
            at = (4 if i == 0 else 1) + t
            if at < len(requests[i]):
                entries.append(StepEntry(slots[i], [requests[i][at]], [0]))
                owners.append(i)
        out = engine.step(entries)
        for row, i in enumerate(owners):
            rows[i].append(out[row:row + 1])
    for i in (0, 1):
        assert_close(torch.cat(rows[i]), toy_oracle(raw, wf, requests[i]), dtype, f"toy model, request {i} step by step")
        engine.release(slots[i])


class ToyDecayMixerOnDevice(ToyDecayMixer):
    """The same recurrence with a one-token step that only launches device work (gather the state rows of the
    step's slots, update, scatter back), so that it may say ``graph_safe`` and its steps are captured in CUDA graphs."""

    graph_safe = True

    def forward(self, x, ctx, cache):
        if not ctx.is_decode:
            return super().forward(x, ctx, cache)
        slots = ctx.slots.long()
        state = self.decay * cache.state.index_select(0, slots) + x.float() @ self.weight.T
        cache.state.index_copy_(0, slots, state)
        return GemmOut(state.to(self.runtime.dtype)[None].contiguous())


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_padded_rows_of_a_captured_step_leave_every_live_state_alone(dtype):
    """Three sequences run as a captured step of four rows; the padded row must not touch the state of the
    sequence in slot 0 (it has a spare state row of its own, as it has a spare cache page)."""
    register_mixer("toy_decay_device", ToyDecayMixerOnDevice)
    register_architecture("ToyForCausalLM", ToyConfig)
    raw = {"architectures": ["ToyForCausalLM"], "hidden_size": 40, "inter": 56, "vocab": 97, "eps": 1e-5, "decay": 0.8,
           "mixer_kind": "toy_decay_device"}
    from qwen_triton_b200.config import config_from_dict
    from qwen_triton_b200.engine.model import expected_tensors
    import json
    config = config_from_dict(raw)
    weights = weights_for(expected_tensors(config.model_spec()), dtype, seed=10)
    with tempfile.TemporaryDirectory() as folder:
        write_safetensors(f"{folder}/model.safetensors", weights)
        with open(f"{folder}/config.json", "w") as handle:
            json.dump(raw, handle)
        engine = Engine.from_pretrained(folder, dtype=dtype, max_tokens=512)
    assert engine._graphs_enabled
    wf = {k: v.float() for k, v in weights.items()}
    requests = [[5, 9, 2, 77, 30, 11, 4, 8, 60], [96, 0, 41, 7, 7, 19, 3], [1, 2, 3, 4, 5, 6, 7, 8]]
    slots = [engine.new_sequence() for _ in requests]
    assert 0 in slots
    prompt = 3
    first = engine.step([StepEntry(slot, tokens[:prompt], [prompt - 1]) for slot, tokens in zip(slots, requests)])
    rows = {i: [first[i:i + 1]] for i in range(3)}
    for at in range(prompt, 7):                                  # four one-token steps: launched, captured, replayed twice
        out = engine.step([StepEntry(slot, [tokens[at]], [0]) for slot, tokens in zip(slots, requests)])
        for i in range(3):
            rows[i].append(out[i:i + 1])
    assert engine.graph_replays >= 2
    for i, tokens in enumerate(requests):
        assert_close(torch.cat(rows[i]), toy_oracle(raw, wf, tokens)[prompt - 1:7], dtype, f"request {i} in slot {slots[i]}")
        engine.release(slots[i])


# ----------------------------------------------------------------------------- a block with two parts that keep something
class ToyTwoBranchBlock:
    """h += attention(norm1(h)) + decay_mixer(norm1(h)); h += feed_forward(norm2(h)): an arrangement with a recurrent
    branch beside the attention, defined here.  It asks the cache for keys/values and for a state block, and gets a
    tuple of two views; its second mixer comes from ``LayerSpec.extra``, as does another norm kind in front of the
    feed-forward."""

    def __init__(self, layer, runtime):
        p = layer.prefix
        self.norm1 = part_class("norm", layer.norm)(layer.norm.params, f"{p}.norm1", runtime)
        second = layer.extra.get("feed_forward_norm", layer.norm)
        self.norm2 = part_class("norm", second)(second.params, f"{p}.norm2", runtime)
        self.attention = part_class("mixer", layer.mixer)(layer.mixer.params, f"{p}.attn", runtime)
        side = layer.extra["side_mixer"]
        self.side = part_class("mixer", side)(side.params, f"{p}.side", runtime)
        self.feed_forward = part_class("feed_forward", layer.feed_forward)(layer.feed_forward.params, f"{p}.ff", runtime)
        self.runtime = runtime

    @classmethod
    def expected_tensors(cls, layer):
        p, out = layer.prefix, {}
        second = layer.extra.get("feed_forward_norm", layer.norm)
        out.update(part_class("norm", layer.norm).expected_tensors(layer.norm.params, f"{p}.norm1"))
        out.update(part_class("norm", second).expected_tensors(second.params, f"{p}.norm2"))
        out.update(part_class("mixer", layer.mixer).expected_tensors(layer.mixer.params, f"{p}.attn"))
        out.update(part_class("mixer", layer.extra["side_mixer"]).expected_tensors(layer.extra["side_mixer"].params, f"{p}.side"))
        out.update(part_class("feed_forward", layer.feed_forward).expected_tensors(layer.feed_forward.params, f"{p}.ff"))
        return out

    graph_safe = True

    def load(self, source):
        for part in (self.norm1, self.norm2, self.attention, self.side, self.feed_forward):
            part.load(source)

    def cache_requests(self):
        return [self.attention.cache_request(), self.side.cache_request()]

    def forward(self, stream, ctx, caches):
        x = self.norm1.apply(stream)
        both = self.attention.forward(x, ctx, caches[0]).value() + self.side.forward(x, ctx, caches[1]).value()
        stream.add(GemmOut(both[None].contiguous()))
        x = self.norm2.apply(stream)
        stream.add(self.feed_forward.forward(x, ctx))


class ToyShiftedNorm:
    """x * rsqrt(mean(x^2) + eps) * (w + 0.5): another norm kind for one of a block's two places."""

    graph_safe = True

    def __init__(self, params, name, runtime):
        self.size, self.eps, self.name, self.runtime = int(params["size"]), float(params["eps"]), name, runtime
        runtime.workspace.declare("toy_shifted", runtime.max_step_tokens * self.size, runtime.dtype)

    @classmethod
    def expected_tensors(cls, params, name):
        return {f"{name}.weight": TensorSpec((int(params["size"]),), role="vector", init_std=0.1, init_mean=1.0)}

    def load(self, source):
        self.weight = (source(f"{self.name}.weight").float() + 0.5).to(self.runtime.device).contiguous()

    def apply(self, stream, rows=None):
        from qwen_triton_b200.ops import kernels
        count = stream.residual.shape[0] if rows is None else rows.shape[0]
        out = self.runtime.workspace.view("toy_shifted", count, self.size)
        kernels.add_rmsnorm(stream.residual, stream.pending, self.weight, self.eps, out, rows)
        if rows is None:
            stream.pending = None
        return out


class TwoBranchConfig(ToyConfig):
    def model_spec(self):
        r = self.raw
        hidden = r["hidden_size"]
        norm = PartSpec("rmsnorm", {"size": hidden, "eps": r["eps"]})
        shifted = PartSpec("toy_shifted_norm", {"size": hidden, "eps": r["eps"]})
        ff = PartSpec("gated_mlp", {"hidden_size": hidden, "intermediate_size": r["inter"], "activation": "relu"})
        attn = PartSpec("attention", {"hidden_size": hidden, "num_heads": 2, "num_kv_heads": 1, "head_dim": 16, "window": None,
                                      "qk_norm": False, "position": PartSpec("none"),
                                      "q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj"})
        side = PartSpec("toy_decay_device", {"hidden_size": hidden, "decay": r["decay"]})
        layer = LayerSpec("blocks.0", PartSpec("toy_two_branch"), attn, ff, norm, extra={"side_mixer": side, "feed_forward_norm": shifted})
        return ModelSpec(architecture="TwoBranchForCausalLM", vocab_size=r["vocab"], hidden_size=hidden,
                         embedding=PartSpec("token_embedding", {"name": "embed.weight"}), layers=(layer,),
                         schedule=(LayerCall(0), LayerCall(0)),
                         final_norm=PartSpec("rmsnorm", {"size": hidden, "eps": r["eps"], "name": "final"}),
                         head=PartSpec("linear_head", {"name": "head.weight", "tied_to": "embed.weight"}), max_positions=256)


def two_branch_oracle(raw, w, tokens):
    hidden, eps, n = raw["hidden_size"], raw["eps"], len(tokens)
    x = w["embed.weight"][torch.tensor(tokens)]
    p = "blocks.0"
    for _ in range(2):                                          # the layer's weights run twice, each call with caches of its own
        h = plain.rms_norm(x, w[f"{p}.norm1.weight"], eps)
        q = (h @ w[f"{p}.attn.q_proj.weight"].T).view(n, 2, 16)
        k = (h @ w[f"{p}.attn.k_proj.weight"].T).view(n, 1, 16)
        v = (h @ w[f"{p}.attn.v_proj.weight"].T).view(n, 1, 16)
        attended = plain.attention_scores(q, k, v, 16 ** -0.5, None).reshape(n, 32) @ w[f"{p}.attn.o_proj.weight"].T
        proj = h @ w[f"{p}.side.mix.weight"].T
        state, side = torch.zeros(hidden), []
        for t in range(n):
            state = raw["decay"] * state + proj[t]
            side.append(state)
        x = x + attended + torch.stack(side)
        h = plain.rms_norm(x, w[f"{p}.norm2.weight"] + 0.5, eps)
        gate, up = h @ w[f"{p}.ff.gate_proj.weight"].T, h @ w[f"{p}.ff.up_proj.weight"].T
        x = x + (torch.relu(gate) * up) @ w[f"{p}.ff.down_proj.weight"].T
    return plain.rms_norm(x, w["final.weight"], eps) @ w["embed.weight"].T


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_a_block_with_two_parts_that_keep_something_and_two_norm_kinds(dtype):
    from qwen_triton_b200.parts import register_block, register_norm
    register_mixer("toy_decay_device", ToyDecayMixerOnDevice)
    register_block("toy_two_branch", ToyTwoBranchBlock)
    register_norm("toy_shifted_norm", ToyShiftedNorm)
    register_architecture("TwoBranchForCausalLM", TwoBranchConfig)
    raw = {"architectures": ["TwoBranchForCausalLM"], "hidden_size": 40, "inter": 48, "vocab": 61, "eps": 1e-5, "decay": 0.7}
    from qwen_triton_b200.config import config_from_dict
    from qwen_triton_b200.engine.model import expected_tensors
    import json
    config = config_from_dict(raw)
    weights = weights_for(expected_tensors(config.model_spec()), dtype, seed=12)
    with tempfile.TemporaryDirectory() as folder:
        write_safetensors(f"{folder}/model.safetensors", weights)
        with open(f"{folder}/config.json", "w") as handle:
            json.dump(raw, handle)
        engine = Engine.from_pretrained(folder, dtype=dtype, max_tokens=512)
    assert len(engine.cache.groups) == 1 and len(engine.cache.groups[0].owners) == 2         # two calls, an attention entry each
    views = engine.cache.view(1)
    assert isinstance(views, tuple) and views[0].k is not None and views[1].state is not None
    wf = {k: v.float() for k, v in weights.items()}
    requests = [[5, 9, 2, 60, 30, 11, 4, 8], [17, 0, 41, 7, 7, 19]]
    slots = [engine.new_sequence() for _ in requests]
    first = engine.step([StepEntry(slots[0], requests[0][:3], [0, 1, 2]), StepEntry(slots[1], requests[1][:2], [0, 1])])
    rows = {0: [first[:3]], 1: [first[3:]]}
    for t in range(5):
        live = [i for i in (0, 1) if (3 if i == 0 else 2) + t < len(requests[i])]
        out = engine.step([StepEntry(slots[i], [requests[i][(3 if i == 0 else 2) + t]], [0]) for i in live])
        for row, i in enumerate(live):
            rows[i].append(out[row:row + 1])
    assert engine.graph_replays >= 2
    for i in (0, 1):
        assert_close(torch.cat(rows[i]), two_branch_oracle(raw, wf, requests[i]), dtype, f"request {i}")
        engine.release(slots[i])
