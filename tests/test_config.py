"""Configuration, registry and spec (no GPU)."""
import json

import pytest

from qwen_triton_b200.config import (ConfigError, LayerCall, ModelSpec, PartSpec, Qwen3Config, config_from_dict,
                                     load_config, load_preset, preset_names, register_architecture,
                                     registered_architectures)

BASE = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=503, hidden_size=96,
            intermediate_size=160, num_hidden_layers=3, num_attention_heads=8)


def test_defaults_follow_the_reference():
    cfg = Qwen3Config.from_hf_config(BASE)
    assert cfg.head_dim == 96 // 8                     # hidden // heads when head_dim is absent
    assert cfg.num_key_value_heads == 8                # defaults to the query heads
    assert cfg.rope_theta == 10000.0 and cfg.rms_norm_eps == 1e-6
    assert cfg.max_position_embeddings == 32768 and not cfg.tie_word_embeddings
    assert cfg.layer_types == ("full_attention",) * 3
    assert cfg.rotary_dim == cfg.head_dim and cfg.eos_token_id == ()


def test_head_dim_is_independent_of_hidden_size():
    cfg = Qwen3Config.from_hf_config({**BASE, "head_dim": 32, "num_key_value_heads": 1})
    assert cfg.q_size == 256 and cfg.kv_size == 32 and cfg.group_size == 8
    spec = cfg.model_spec()
    mixer = spec.layers[0].mixer
    assert mixer["head_dim"] == 32 and mixer["scale"] == 32 ** -0.5 and mixer["num_kv_heads"] == 1


def test_rope_theta_under_rope_parameters_and_text_config():
    cfg = Qwen3Config.from_hf_config({**BASE, "rope_parameters": {"rope_theta": 5e5, "rope_type": "default"}})
    assert cfg.rope_theta == 5e5
    wrapped = {"architectures": ["Qwen3ForCausalLM"], "tie_word_embeddings": True,
               "text_config": {**BASE, "tie_word_embeddings": False}}
    assert Qwen3Config.from_hf_config(wrapped).tie_word_embeddings is True     # top level wins


def test_eos_may_be_a_list():
    assert Qwen3Config.from_hf_config({**BASE, "eos_token_id": [5, 6]}).eos_token_id == (5, 6)
    assert Qwen3Config.from_hf_config({**BASE, "eos_token_id": 7}).model_spec().eos_token_ids == (7,)


def test_sliding_window_layers_from_max_window_layers():
    cfg = Qwen3Config.from_hf_config({**BASE, "use_sliding_window": True, "sliding_window": 16, "max_window_layers": 1})
    assert cfg.layer_types == ("full_attention", "sliding_attention", "sliding_attention")
    windows = [layer.mixer["window"] for layer in cfg.model_spec().layers]
    assert windows == [None, 16, 16]
    # a window that is configured but switched off changes nothing
    off = Qwen3Config.from_hf_config({**BASE, "use_sliding_window": False, "sliding_window": 16})
    assert off.layer_types == ("full_attention",) * 3


@pytest.mark.parametrize("patch, word", [
    ({"model_type": "qwen3_moe"}, "model_type"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"hidden_act": "gelu"}, "SiLU"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "rope scaling"),
    ({"head_dim": 15}, "even"),
    ({"layer_types": ["full_attention", "linear_attention", "full_attention"]}, "linear_attention"),
    ({"layer_types": ["full_attention"]}, "entries"),
    ({"use_sliding_window": True, "layer_types": ["sliding_attention"] * 3}, "sliding_window"),
    ({"vocab_size": None}, "vocab_size"),
])
def test_what_is_not_built_is_refused(patch, word):
    with pytest.raises(ConfigError, match=word):
        Qwen3Config.from_hf_config({**BASE, **patch})


def test_registry_picks_the_class_by_architecture_name():
    assert "Qwen3ForCausalLM" in registered_architectures()
    assert isinstance(config_from_dict(BASE), Qwen3Config)
    no_names = {k: v for k, v in BASE.items() if k != "architectures"}
    assert isinstance(config_from_dict(no_names), Qwen3Config)          # falls back to model_type
    with pytest.raises(KeyError, match="Qwen3ForCausalLM"):
        config_from_dict({**BASE, "architectures": ["LlamaForCausalLM"]})
    with pytest.raises(ValueError, match="already registered"):
        register_architecture("Qwen3ForCausalLM", dict)


def test_round_trip_through_config_json(tmp_path):
    cfg = load_preset("tiny-c")
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_hf_dict()))
    again = load_config(tmp_path)
    assert again == cfg
    # layer types that no cutoff describes survive the trip as the list they are
    mixed = Qwen3Config.from_hf_config({**BASE, "sliding_window": 16,
                                        "layer_types": ["sliding_attention", "full_attention", "sliding_attention"]})
    (tmp_path / "config.json").write_text(json.dumps(mixed.to_hf_dict()))
    assert load_config(tmp_path).layer_types == ("sliding_attention", "full_attention", "sliding_attention")


def test_presets_differ_in_every_size_and_option():
    a, b, c, d = (load_preset(n) for n in ("tiny-a", "tiny-b", "tiny-c", "tiny-d"))
    for field in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "head_dim", "rope_theta", "rms_norm_eps"):
        assert len({getattr(a, field), getattr(b, field), getattr(c, field), getattr(d, field)}) == 4, field
    assert a.tie_word_embeddings and not b.tie_word_embeddings
    assert d.attention_bias and not (a.attention_bias or b.attention_bias or c.attention_bias)
    assert b.q_size != b.hidden_size and c.use_sliding_window and not a.use_sliding_window
    assert {"qwen3-0.6b", "qwen3-8b", "qwen3-32b"} <= set(preset_names())
    big = load_preset("qwen3-8b")
    assert (big.num_hidden_layers, big.hidden_size, big.intermediate_size, big.vocab_size) == (36, 4096, 12288, 151936)


def test_schedule_is_data_and_is_checked():
    spec = load_preset("tiny-a").model_spec()
    assert [c.layer for c in spec.schedule] == [0, 1] and all(c.cache_of is None for c in spec.schedule)
    fields = {f: getattr(spec, f) for f in spec.__dataclass_fields__}
    twice = ModelSpec(**{**fields, "schedule": (LayerCall(0), LayerCall(1), LayerCall(0), LayerCall(1, cache_of=1))})
    twice.validate()
    for bad in ((LayerCall(2),), (LayerCall(0, cache_of=0),), (LayerCall(0), LayerCall(1, cache_of=0), LayerCall(0, cache_of=1))):
        with pytest.raises(ValueError):
            ModelSpec(**{**fields, "schedule": bad}).validate()
    assert PartSpec("x", {"a": 1})["a"] == 1


def test_attention_bias_adds_the_four_bias_tensors():
    from qwen_triton_b200.engine.model import expected_tensors
    biased, plain = (expected_tensors(load_preset(n).model_spec()) for n in ("tiny-d", "tiny-a"))
    cfg = load_preset("tiny-d")
    for name, rows in (("q_proj", cfg.q_size), ("k_proj", cfg.num_key_value_heads * cfg.head_dim),
                       ("v_proj", cfg.num_key_value_heads * cfg.head_dim), ("o_proj", cfg.hidden_size)):
        for layer in range(cfg.num_hidden_layers):
            assert tuple(biased[f"model.layers.{layer}.self_attn.{name}.bias"].shape) == (rows,)
    assert not any(name.endswith(".bias") for name in plain)
