"""One registry from an architecture's name (config.json `architectures[0]`) to what the
engine needs of it: its typed configuration class and a function that turns that
configuration into an architecture-neutral `ModelSpec`.

The reference has no registry: it checks `model_type == "qwen2"` and constructs its
single model class (src/model/huggingface.cpp:152-154).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict

from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any                       # has from_dict / from_json / to_dict / validate
    build_spec: Callable[[Any], ModelSpec]  # typed config -> ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture, *, replace: bool = False) -> None:
    if arch.name in _ARCHITECTURES and not replace:
        raise KeyError(f"architecture {arch.name!r} is already registered")
    _ARCHITECTURES[arch.name] = arch


def get_architecture(name: str) -> Architecture:
    _ensure_builtin()
    if name not in _ARCHITECTURES:
        raise KeyError(f"unknown architecture {name!r}; registered: {', '.join(sorted(_ARCHITECTURES))}")
    return _ARCHITECTURES[name]


def architectures() -> Dict[str, Architecture]:
    _ensure_builtin()
    return dict(_ARCHITECTURES)


def architecture_of(raw_config: Dict[str, Any]) -> Architecture:
    """Choose the architecture from a parsed config.json."""
    _ensure_builtin()
    names = raw_config.get("architectures") or []
    for n in names:
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    # Files written by hand for the reference carry only model_type (its parser needs no
    # `architectures`); accept that spelling for the one family it has.
    if not names and raw_config.get("model_type") == "qwen2":
        return _ARCHITECTURES["Qwen2ForCausalLM"]
    raise KeyError(f"config.json names architectures {names!r}; registered: "
                   f"{', '.join(sorted(_ARCHITECTURES))}")


def load_config(folder_or_file: str):
    """Read config.json and return (architecture, typed config)."""
    path = folder_or_file
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    with open(path, "r", encoding="utf-8") as f:
        raw = json.load(f)
    arch = architecture_of(raw)
    return arch, arch.config_class.from_dict(raw)


_loaded = False


def _ensure_builtin() -> None:
    global _loaded
    if not _loaded:
        _loaded = True
        from ..models import qwen2  # noqa: F401  (registers itself)
