"""One registry from an architecture's name (config.json `architectures[0]`) to what the
engine needs of it: its typed configuration class and a function that turns that
configuration into an architecture-neutral `ModelSpec`.

The reference has no registry: it checks `model_type == "qwen2"` and constructs its
single model class (src/model/huggingface.cpp:152-154).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Tuple

from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any                       # has from_dict / from_json / to_dict / validate
    build_spec: Callable[[Any], ModelSpec]  # typed config -> ModelSpec
    # config.json files without `architectures` are matched by their `model_type` against these spellings
    model_types: Tuple[str, ...] = ()
    # named configurations (name -> config.json keys) that `preset()` and the command line's --random-config offer
    presets: Dict[str, Dict[str, Any]] = field(default_factory=dict, hash=False, compare=False)


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
    # `architectures`); an architecture may register the spellings it answers to.
    if not names and raw_config.get("model_type"):
        for arch in _ARCHITECTURES.values():
            if raw_config["model_type"] in arch.model_types:
                return arch
    raise KeyError(f"config.json names architectures {names!r}; registered: "
                   f"{', '.join(sorted(_ARCHITECTURES))}")


def architecture_for(config) -> Architecture:
    """The architecture a typed configuration object belongs to."""
    _ensure_builtin()
    for arch in _ARCHITECTURES.values():
        if type(config) is arch.config_class:
            return arch
    raise KeyError(f"no registered architecture has the configuration class {type(config).__name__}")


def find_preset(name: str, **overrides):
    """(architecture, typed config) of a named preset of any registered architecture."""
    _ensure_builtin()
    known = []
    for arch in _ARCHITECTURES.values():
        known += list(arch.presets)
        if name in arch.presets:
            raw = dict(arch.presets[name])
            raw.update(overrides)
            return arch, arch.config_class.from_dict(raw)
    raise KeyError(f"unknown preset {name!r}; known: {', '.join(sorted(known))}")


def parameter_count(arch: Architecture, config) -> int:
    """Elements of every tensor the model declares (a tied head counts once): from the parts' own declarations,
    so it holds for any architecture."""
    import torch

    from ..parts.base import Runtime
    from ..parts.build import build_model
    model = build_model(arch.build_spec(config), Runtime(torch.device("cpu"), torch.float32))
    total = 0
    for spec in model.expected_tensors().values():
        n = 1
        for s in spec.shape:
            n *= int(s)
        total += n
    return total


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
