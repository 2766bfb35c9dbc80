"""Weights by name: round trip, name normalisation, and the one error that lists every fault (no GPU)."""
import json

import pytest
import torch

from qwen_triton_b200.config import load_preset
from qwen_triton_b200.engine.model import expected_tensors
from qwen_triton_b200.weights.tensors import TensorSpec
from qwen_triton_b200.weights import (Checkpoint, WeightsError, kept_dtype, open_checkpoint, random_tensor,
                                      write_random_model, write_safetensors)


def _tensors(folder):
    checkpoint = Checkpoint(folder)
    return {name: checkpoint.read(name) for name in checkpoint.names()}


def test_random_model_folder_round_trip(tmp_path):
    config = load_preset("tiny-b")
    write_random_model(tmp_path, config, seed=1, dtype=torch.bfloat16)
    expected = expected_tensors(config.model_spec())
    source = open_checkpoint(tmp_path, expected)
    assert json.loads((tmp_path / "config.json").read_text())["torch_dtype"] == "bfloat16"
    for name, spec in expected.items():
        tensor = source(name)
        assert tuple(tensor.shape) == spec.shape and tensor.dtype == torch.bfloat16
        assert torch.equal(tensor, random_tensor(name, spec, 1, torch.bfloat16))
    norm = source("model.layers.0.input_layernorm.weight").float()
    assert 0.5 < float(norm.mean()) < 1.5 and float(norm.std()) > 0.03        # norm weights are not all ones
    # safetensors' own reader agrees with ours
    from safetensors import safe_open
    with safe_open(str(tmp_path / "model.safetensors"), framework="pt") as handle:
        assert torch.equal(handle.get_tensor("lm_head.weight"), source("lm_head.weight"))


def test_values_depend_on_seed_and_name_only(tmp_path):
    config = load_preset("tiny-a")
    a = _tensors(write_random_model(tmp_path / "a", config, 0, torch.float32))
    b = _tensors(write_random_model(tmp_path / "b", config, 0, torch.float32))
    c = _tensors(write_random_model(tmp_path / "c", config, 1, torch.float32))
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.norm.weight"], c["model.norm.weight"])
    assert "lm_head.weight" not in a                                          # tied: the head is the embedding


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    config = load_preset("tiny-a")
    tensors = _tensors(write_random_model(tmp_path / "ok", config, 0, torch.float32))
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 63)
    bad = tmp_path / "bad"
    bad.mkdir()
    write_safetensors(bad / "model.safetensors", tensors)
    with pytest.raises(WeightsError) as caught:
        open_checkpoint(bad, expected_tensors(config.model_spec()))
    error = caught.value
    assert error.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert error.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert len(error.wrong_shape) == 1 and "(64, 63)" in error.wrong_shape[0] and "(64, 64)" in error.wrong_shape[0]
    text = str(error)
    for word in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "up_proj", "inv_freq", "q_proj"):
        assert word in text


def test_wrapped_names_and_shards(tmp_path):
    config = load_preset("tiny-a")
    tensors = _tensors(write_random_model(tmp_path / "ok", config, 0, torch.float32))
    wrapped = {("model.language_model." + k[len("model."):]) if k.startswith("model.") else k: v for k, v in tensors.items()}
    names = sorted(wrapped)
    shard_dir = tmp_path / "shards"
    shard_dir.mkdir()
    half = len(names) // 2
    write_safetensors(shard_dir / "model-00001-of-00002.safetensors", {k: wrapped[k] for k in names[:half]})
    write_safetensors(shard_dir / "model-00002-of-00002.safetensors", {k: wrapped[k] for k in names[half:]})
    weight_map = {k: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
                  for i, k in enumerate(names)}
    (shard_dir / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    (shard_dir / "stray.safetensors").write_bytes(b"")                       # not in the index: must be ignored
    source = open_checkpoint(shard_dir, expected_tensors(config.model_spec()))
    assert torch.equal(source("model.layers.1.self_attn.k_norm.weight"), tensors["model.layers.1.self_attn.k_norm.weight"])


def test_tied_model_reads_past_a_stored_head(tmp_path):
    config = load_preset("tiny-a")
    tensors = _tensors(write_random_model(tmp_path / "ok", config, 0, torch.float32))
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    tied = tmp_path / "tied"
    tied.mkdir()
    write_safetensors(tied / "model.safetensors", tensors)
    open_checkpoint(tied, expected_tensors(config.model_spec()))             # no error
    untied = load_preset("tiny-b")
    with pytest.raises(WeightsError, match="lm_head.weight"):
        stripped = _tensors(write_random_model(tmp_path / "b", untied, 0, torch.float32))
        del stripped["lm_head.weight"]
        target = tmp_path / "b2"
        target.mkdir()
        write_safetensors(target / "model.safetensors", stripped)
        open_checkpoint(target, expected_tensors(untied.model_spec()))


def test_missing_folder_and_kept_precisions(tmp_path):
    config = load_preset("tiny-a")
    with pytest.raises(FileNotFoundError):
        open_checkpoint(tmp_path, expected_tensors(config.model_spec()))
    expected = expected_tensors(config.model_spec())
    assert kept_dtype(expected["model.norm.weight"], torch.bfloat16) == torch.float32       # vectors stay 32-bit
    assert kept_dtype(expected["model.embed_tokens.weight"], torch.bfloat16) == torch.bfloat16
    assert kept_dtype(expected["model.embed_tokens.weight"], torch.float32) == torch.float32


def test_random_draw_is_the_stated_integer_recipe():
    """Element i = (sum of the twelve 16-bit fields of splitmix64 outputs 3i+1..3i+3 of the tensor's stream - 393210) / 65536,
    restated here in plain Python integers."""
    from qwen_triton_b200.weights.random_init import _tensor_seed, standard_normal
    mask = (1 << 64) - 1

    def mix(v):
        v = ((v ^ (v >> 30)) * 0xBF58476D1CE4E5B9) & mask
        v = ((v ^ (v >> 27)) * 0x94D049BB133111EB) & mask
        return v ^ (v >> 31)

    def element(stream, i):
        total = 0
        for j in range(3):
            word = mix(((3 * i + j + 1) * 0x9E3779B97F4A7C15 + stream) & mask)
            total += sum((word >> (16 * f)) & 0xFFFF for f in range(4))
        return (total - 393210) / 65536.0

    stream = _tensor_seed(4, "model.norm.weight")
    drawn = standard_normal(stream, 1000, 64)
    assert drawn.tolist() == [element(stream, i) for i in range(1000, 1064)]
    many = standard_normal(stream, 0, 1 << 18)
    assert abs(float(many.mean())) < 0.01 and abs(float(many.std()) - 1.0) < 0.01
    # a tensor is the same whether it is drawn in one piece or in several
    spec = TensorSpec((3, 50), init_std=0.02)
    whole = random_tensor("w", spec, 9, torch.float32)
    assert torch.equal(whole.flatten()[37:91], standard_normal(_tensor_seed(9, "w"), 37, 54) * 0.02 + 0.0)
    # stored in bfloat16, computed in float32: the bfloat16 values, exactly
    assert torch.equal(random_tensor("w", spec, 9, torch.float32, store_dtype=torch.bfloat16),
                       random_tensor("w", spec, 9, torch.bfloat16).float())
