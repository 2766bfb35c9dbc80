"""Typed configuration of the Qwen3 dense architecture, read from config.json.

Keys, defaults and derived values follow the reference's normalisation
(qwen_triton/configs/config.py:111-200): ``head_dim`` defaults to
``hidden_size // num_attention_heads`` (:139) but is independent of it when
given, ``num_key_value_heads`` defaults to the number of query heads (:158),
``rope_theta`` may sit at top level or under ``rope_parameters`` (:140-144),
``tie_word_embeddings`` at top level wins over ``text_config`` (:165), and
layers at index >= ``max_window_layers`` use the sliding window when
``use_sliding_window`` is set (:22-27).  Only ``model_type == "qwen3"`` is
accepted (family ``qwen3_dense``, :35-36).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Mapping

from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec

FULL_ATTENTION = "full_attention"
SLIDING_ATTENTION = "sliding_attention"


class ConfigError(ValueError):
    """config.json asks for something this library does not build."""


def _as_int_tuple(value: Any) -> tuple[int, ...]:
    if value is None:
        return ()
    if isinstance(value, (list, tuple)):
        return tuple(int(v) for v in value)
    return (int(value),)


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    hidden_act: str = "silu"
    max_position_embeddings: int = 32768
    initializer_range: float = 0.02
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    rope_theta: float = 10000.0
    partial_rotary_factor: float = 1.0
    attention_bias: bool = False
    use_sliding_window: bool = False
    sliding_window: int | None = None
    max_window_layers: int | None = None
    layer_types: tuple[str, ...] = ()
    pad_token_id: int | None = None
    bos_token_id: int | None = None
    eos_token_id: tuple[int, ...] = ()
    torch_dtype: str = ""
    model_type: str = "qwen3"
    architectures: tuple[str, ...] = ("Qwen3ForCausalLM",)
    raw: Mapping[str, Any] = field(default_factory=dict, repr=False, compare=False)

    family = "qwen3_dense"

    # ------------------------------------------------------------------ derived
    @property
    def rotary_dim(self) -> int:
        """Even, at least 2 (qwen_triton/configs/config.py:103-109)."""
        rd = max(2, int(self.head_dim * self.partial_rotary_factor))
        return rd - (rd % 2)

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_hf_config(cls, hf_config: Mapping[str, Any] | str | Path) -> "Qwen3Config":
        """Accepts the config.json mapping, a model folder or a path to config.json."""
        if isinstance(hf_config, (str, Path)):
            path = Path(hf_config)
            path = path / "config.json" if path.is_dir() else path
            with path.open("r", encoding="utf-8") as handle:
                hf_config = json.load(handle)
        if hasattr(hf_config, "to_dict"):
            hf_config = hf_config.to_dict()
        if not isinstance(hf_config, Mapping):
            raise TypeError(f"unsupported config type: {type(hf_config)!r}")
        raw = dict(hf_config)
        text = dict(raw.get("text_config") or raw)

        model_type = str(text.get("model_type") or raw.get("model_type"))
        if model_type != "qwen3":
            raise ConfigError(f"Qwen3Config reads model_type 'qwen3', not {model_type!r}")
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads"):
            if text.get(key) is None:
                raise ConfigError(f"config.json lacks the key {key!r}")

        rope_params = dict(text.get("rope_parameters") or {})
        scaling = text.get("rope_scaling")
        scaling_kind = scaling.get("rope_type", scaling.get("type")) if isinstance(scaling, Mapping) else scaling
        for value in (scaling_kind, rope_params.get("rope_type")):
            if value not in (None, "default"):
                raise ConfigError(f"rope scaling of type {value!r} is not part of this architecture's position encoding")

        num_layers = int(text["num_hidden_layers"])
        heads = int(text["num_attention_heads"])
        hidden = int(text["hidden_size"])
        use_window = bool(text.get("use_sliding_window", False))
        window = text.get("sliding_window")
        max_window_layers = text.get("max_window_layers")
        layer_types = text.get("layer_types")
        if layer_types:
            layer_types = tuple(str(t) for t in layer_types)
        elif use_window and window is not None:
            cutoff = int(max_window_layers) if max_window_layers is not None else num_layers
            layer_types = tuple(SLIDING_ATTENTION if i >= cutoff else FULL_ATTENTION for i in range(num_layers))
        else:
            layer_types = (FULL_ATTENTION,) * num_layers

        config = cls(
            vocab_size=int(text["vocab_size"]),
            hidden_size=hidden,
            intermediate_size=int(text["intermediate_size"]),
            num_hidden_layers=num_layers,
            num_attention_heads=heads,
            num_key_value_heads=int(text.get("num_key_value_heads") or heads),
            head_dim=int(text.get("head_dim") or hidden // heads),
            hidden_act=str(text.get("hidden_act", "silu")),
            max_position_embeddings=int(text.get("max_position_embeddings", 32768)),
            initializer_range=float(text.get("initializer_range", 0.02)),
            rms_norm_eps=float(text.get("rms_norm_eps", 1e-6)),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", text.get("tie_word_embeddings", False))),
            rope_theta=float(text.get("rope_theta") or rope_params.get("rope_theta") or 10000.0),
            partial_rotary_factor=float(
                text.get("partial_rotary_factor") or rope_params.get("partial_rotary_factor") or 1.0
            ),
            attention_bias=bool(text.get("attention_bias", False)),
            use_sliding_window=use_window,
            sliding_window=int(window) if window is not None else None,
            max_window_layers=int(max_window_layers) if max_window_layers is not None else None,
            layer_types=layer_types,
            pad_token_id=text.get("pad_token_id", raw.get("pad_token_id")),
            bos_token_id=text.get("bos_token_id", raw.get("bos_token_id")),
            eos_token_id=_as_int_tuple(text.get("eos_token_id", raw.get("eos_token_id"))),
            torch_dtype=str(text.get("torch_dtype") or text.get("dtype") or raw.get("torch_dtype") or ""),
            model_type=model_type,
            architectures=tuple(raw.get("architectures") or ("Qwen3ForCausalLM",)),
            raw=raw,
        )
        config.validate()
        return config

    def validate(self) -> None:
        problems: list[str] = []
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings"):
            if getattr(self, name) <= 0:
                problems.append(f"{name} must be positive, got {getattr(self, name)}")
        if not problems and self.num_attention_heads % self.num_key_value_heads:
            problems.append(
                f"num_attention_heads={self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads={self.num_key_value_heads}"
            )
        if self.head_dim % 2:
            problems.append(f"head_dim={self.head_dim} must be even for rotate-half position encoding")
        if self.hidden_act != "silu":
            problems.append(f"hidden_act={self.hidden_act!r}: the feed-forward of this architecture is SiLU-gated")
        if not (0.0 < self.partial_rotary_factor <= 1.0):
            problems.append(f"partial_rotary_factor={self.partial_rotary_factor} must lie in (0, 1]")
        if self.rms_norm_eps <= 0.0 or self.rope_theta <= 0.0:
            problems.append("rms_norm_eps and rope_theta must be positive")
        if len(self.layer_types) != self.num_hidden_layers:
            problems.append(f"layer_types has {len(self.layer_types)} entries for {self.num_hidden_layers} layers")
        for kind in self.layer_types:
            if kind not in (FULL_ATTENTION, SLIDING_ATTENTION):
                problems.append(f"layer type {kind!r} does not belong to the Qwen3 dense architecture")
        if SLIDING_ATTENTION in self.layer_types and (self.sliding_window is None or self.sliding_window <= 0):
            problems.append("sliding_attention layers need a positive sliding_window")
        if problems:
            raise ConfigError("invalid Qwen3 configuration: " + "; ".join(problems))

    # ------------------------------------------------------------------ export
    def to_hf_dict(self) -> dict[str, Any]:
        """The config.json that parses back into this configuration."""
        out: dict[str, Any] = {
            "architectures": list(self.architectures),
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "hidden_act": self.hidden_act,
            "max_position_embeddings": self.max_position_embeddings,
            "initializer_range": self.initializer_range,
            "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings,
            "rope_theta": self.rope_theta,
            "attention_bias": self.attention_bias,
            "use_sliding_window": self.use_sliding_window,
            "sliding_window": self.sliding_window,
            "max_window_layers": self.max_window_layers,
            "layer_types": list(self.layer_types),
        }
        if self.partial_rotary_factor != 1.0:
            out["partial_rotary_factor"] = self.partial_rotary_factor
        if self.eos_token_id:
            out["eos_token_id"] = self.eos_token_id[0] if len(self.eos_token_id) == 1 else list(self.eos_token_id)
        for key in ("pad_token_id", "bos_token_id"):
            if getattr(self, key) is not None:
                out[key] = getattr(self, key)
        if self.torch_dtype:
            out["torch_dtype"] = self.torch_dtype
        return out

    def model_spec(self) -> ModelSpec:
        """Translate into parts: embedding, pre-norm blocks of (attention, gated MLP), norm, head."""
        position = PartSpec("rope", {"theta": self.rope_theta, "rotary_dim": self.rotary_dim, "head_dim": self.head_dim})
        norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.rms_norm_eps})
        feed_forward = PartSpec("gated_mlp", {
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "activation": self.hidden_act,
            "gate": "gate_proj", "up": "up_proj", "down": "down_proj",
        })
        block = PartSpec("pre_norm", {
            "mixer": "self_attn", "feed_forward": "mlp",
            "mixer_norm": "input_layernorm", "feed_forward_norm": "post_attention_layernorm",
        })
        layers = []
        for index, kind in enumerate(self.layer_types):
            mixer = PartSpec("attention", {
                "hidden_size": self.hidden_size,
                "num_heads": self.num_attention_heads,
                "num_kv_heads": self.num_key_value_heads,
                "head_dim": self.head_dim,
                "scale": self.head_dim ** -0.5,
                "window": self.sliding_window if kind == SLIDING_ATTENTION else None,
                "qk_norm": True,
                "qk_norm_eps": self.rms_norm_eps,
                "bias": self.attention_bias,
                "position": position,
                "q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj",
                "q_norm": "q_norm", "k_norm": "k_norm",
            })
            layers.append(LayerSpec(prefix=f"model.layers.{index}", block=block, mixer=mixer,
                                    feed_forward=feed_forward, norm=norm))
        spec = ModelSpec(
            architecture=self.architectures[0],
            vocab_size=self.vocab_size,
            hidden_size=self.hidden_size,
            embedding=PartSpec("token_embedding", {"name": "model.embed_tokens.weight",
                                                   "init_std": self.initializer_range}),
            layers=tuple(layers),
            schedule=tuple(LayerCall(layer=i) for i in range(self.num_hidden_layers)),
            final_norm=PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.rms_norm_eps,
                                            "name": "model.norm"}),
            head=PartSpec("linear_head", {"name": "lm_head.weight",
                                          "tied_to": "model.embed_tokens.weight" if self.tie_word_embeddings else None}),
            max_positions=self.max_position_embeddings,
            eos_token_ids=self.eos_token_id,
        )
        spec.validate()
        return spec
