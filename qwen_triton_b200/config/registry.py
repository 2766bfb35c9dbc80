"""One registry from an architecture's name to its configuration class.

``config.json`` names its model class under ``architectures``; that name (or,
failing that, ``model_type``) selects the typed configuration, whose
``model_spec()`` describes the model in parts.  The reference has no registry:
one class switches on the family string (qwen_triton/models/core.py:108-116).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Mapping, Protocol


class ArchitectureConfig(Protocol):
    @classmethod
    def from_hf_config(cls, hf_config: Mapping[str, Any]) -> "ArchitectureConfig": ...
    def model_spec(self): ...
    def to_hf_dict(self) -> dict[str, Any]: ...


_BY_ARCHITECTURE: dict[str, type] = {}
_BY_MODEL_TYPE: dict[str, type] = {}


def register_architecture(name: str, config_cls: type, model_type: str | None = None) -> None:
    """Register ``config_cls`` under the class name found in config.json's ``architectures``."""
    if name in _BY_ARCHITECTURE and _BY_ARCHITECTURE[name] is not config_cls:
        raise ValueError(f"architecture {name!r} is already registered")
    _BY_ARCHITECTURE[name] = config_cls
    if model_type is not None:
        _BY_MODEL_TYPE[model_type] = config_cls


def registered_architectures() -> list[str]:
    return sorted(_BY_ARCHITECTURE)


def load_config_dict(model_path: str | Path) -> dict[str, Any]:
    """Read config.json from a model folder (or the file itself)."""
    path = Path(model_path)
    path = path / "config.json" if path.is_dir() else path
    if not path.exists():
        raise FileNotFoundError(f"no config.json at {path}")
    with path.open("r", encoding="utf-8") as handle:
        return json.load(handle)


def config_from_dict(raw: Mapping[str, Any]):
    """Pick the configuration class by ``architectures[0]``, else ``model_type``."""
    names = list(raw.get("architectures") or [])
    for name in names:
        if name in _BY_ARCHITECTURE:
            return _BY_ARCHITECTURE[name].from_hf_config(raw)
    text = raw.get("text_config") or raw
    model_type = text.get("model_type") or raw.get("model_type")
    if not names and model_type in _BY_MODEL_TYPE:
        return _BY_MODEL_TYPE[model_type].from_hf_config(raw)
    raise KeyError(
        f"no registered architecture for architectures={names!r} model_type={model_type!r}; "
        f"registered: {registered_architectures()}"
    )


def load_config(model_path: str | Path):
    return config_from_dict(load_config_dict(model_path))


def preset_names() -> list[str]:
    return sorted(p.stem for p in (Path(__file__).parent / "presets").glob("*.json"))


def load_preset(name: str):
    path = Path(__file__).parent / "presets" / f"{name}.json"
    if not path.exists():
        raise KeyError(f"unknown preset {name!r}; presets: {preset_names()}")
    return load_config(path)
