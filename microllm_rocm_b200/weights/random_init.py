"""Random-weights mode: fill a model from a configuration and a seed, in memory or as a
model folder (config.json + model.safetensors).

Distributions: every matrix, table and bias N(0, 0.02); norm weights 1 + N(0, 0.1); each
part states its own in `WeightSpec.init`.  Each tensor has its own generator seeded from
(seed, tensor name), so a tensor's values do not depend on which other tensors exist or on
the order they are drawn in.  (The reference initialises with std::mt19937_64 and
std::normal_distribution in construction order, src/model/model.cpp:232-237,285-295 --
not reproducible outside one standard library; its biases start at 0 and norms at 1.)
"""
from __future__ import annotations

import os
import zlib
from typing import Dict

import torch

from ..config.registry import Architecture
from ..parts.base import Runtime, WeightSpec
from ..parts.build import build_model
from .loader import target_dtype
from .safetensors import save_file


def _tensor_seed(seed: int, name: str) -> int:
    return (int(seed) * 1000003 + zlib.crc32(name.encode("utf-8"))) % (2 ** 63 - 1)


def draw(spec: WeightSpec, seed: int, name: str, device: torch.device) -> torch.Tensor:
    """fp32 values of one tensor.  CPU and CUDA generators differ: a model folder is always
    written from CPU draws; in-memory models for benchmarks may draw on the device."""
    gen = torch.Generator(device=device)
    gen.manual_seed(_tensor_seed(seed, name))
    kind, std = spec.init
    if spec.role == "int_table":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    x = torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device) * std
    if kind == "one_plus_normal":
        x += 1.0
    elif kind != "normal":
        raise ValueError(f"unknown init {kind!r} for {name}")
    return x


def random_tensors(expected: Dict[str, WeightSpec], seed: int, device: torch.device,
                   storage_dtype: torch.dtype) -> Dict[str, torch.Tensor]:
    """Full name -> tensor as a checkpoint would store it: floating tensors in
    `storage_dtype` (values drawn in fp32, then rounded to nearest even)."""
    out = {}
    for name, spec in expected.items():
        t = draw(spec, seed, name, device)
        out[name] = t if spec.role == "int_table" else t.to(storage_dtype)
    return out


def init_random(model, seed: int, storage_dtype: torch.dtype = None, draw_on_device: bool = False) -> None:
    """Bind random weights to `model` in memory.  Values are those a folder written by
    `write_random_model` with the same seed and storage dtype would hold when
    draw_on_device is False."""
    rt: Runtime = model.rt
    storage_dtype = storage_dtype or rt.dtype
    where = rt.device if draw_on_device else torch.device("cpu")
    expected = model.expected_tensors()
    tensors = {}
    for name, spec in expected.items():
        t = draw(spec, seed, name, where)
        if spec.role != "int_table":
            t = t.to(storage_dtype)
        tensors[name] = t.to(device=rt.device, dtype=target_dtype(spec.role, rt)).contiguous()
    model.bind(tensors)


_DTYPE_NAMES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


def write_random_model(arch: Architecture, config, seed: int, folder: str, storage_dtype: str = None) -> str:
    """Write `folder/config.json` and `folder/model.safetensors` for `config` with weights
    drawn from `seed`.  `storage_dtype` defaults to the configuration's torch_dtype."""
    name = storage_dtype or getattr(config, "torch_dtype", "bfloat16")
    if name not in _DTYPE_NAMES:
        raise ValueError(f"storage dtype {name!r} is not one of {', '.join(_DTYPE_NAMES)}")
    os.makedirs(folder, exist_ok=True)
    raw = config.to_dict()
    raw["torch_dtype"] = name
    import json
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(raw, f, indent=1)
    # only the declarations are needed; build the parts on the CPU, in fp32, without kernels
    model = build_model(arch.build_spec(config), Runtime(torch.device("cpu"), torch.float32))
    tensors = random_tensors(model.expected_tensors(), seed, torch.device("cpu"), _DTYPE_NAMES[name])
    save_file(tensors, os.path.join(folder, "model.safetensors"), metadata={"format": "pt", "seed": str(seed)})
    return folder
