"""Random-weights mode: fill a model from a configuration and a seed, in memory or as a
model folder (config.json + model.safetensors).

Distributions: every matrix, table and bias N(0, 0.02); norm weights 1 + N(0, 0.1); each
part states its own in `WeightSpec.init`.  (The reference initialises with std::mt19937_64 and
std::normal_distribution in construction order, src/model/model.cpp:232-237,285-295 --
not reproducible outside one standard library; its biases start at 0 and norms at 1.)

The generator is counter-based and uses integer arithmetic only, so that the CPU, the GPU and any
other program that restates these few lines produce the same bits, and a large model can be filled
on the device: element i of a tensor takes the three 64-bit words
    SplitMix64 finaliser(key + GOLDEN * (3 i + j + 1)),  j = 0, 1, 2,    key = f(seed, crc32(name)),
cuts them into twelve 16-bit fields, and the standard normal value is (2 * sum - 12 * 65535) / 2^17:
the sum of twelve uniforms (Irwin-Hall; variance 1 - 2^-32, support +-6), exact in fp32.  One fp32
multiplication by the standard deviation (and one addition of 1 for norm weights) follows; a bf16 model
is the round-to-nearest-even of these fp32 values.  A tensor's values depend on (seed, its name, the
element's index) alone: not on which other tensors exist, nor on the order or the device they are drawn on.
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


_GOLDEN = 0x9E3779B97F4A7C15
_MUL1 = 0xBF58476D1CE4E5B9
_MUL2 = 0x94D049BB133111EB
_CHUNK = 1 << 24                  # elements drawn at a time (bounds the integer temporaries to ~1 GB)


def _signed(v: int) -> int:
    """The int64 with the bit pattern of the unsigned 64-bit v (torch has no uint64 arithmetic;
    two's-complement multiplication and addition wrap the same way)."""
    v &= (1 << 64) - 1
    return v - (1 << 64) if v >= (1 << 63) else v


def _shift_right(z: torch.Tensor, bits: int) -> torch.Tensor:
    return (z >> bits) & ((1 << (64 - bits)) - 1)              # logical, not arithmetic


def _finalise(z: torch.Tensor) -> torch.Tensor:
    """SplitMix64's output function on int64 tensors."""
    z = (z ^ _shift_right(z, 30)) * _signed(_MUL1)
    z = (z ^ _shift_right(z, 27)) * _signed(_MUL2)
    return z ^ _shift_right(z, 31)


def tensor_key(seed: int, name: str) -> int:
    """64-bit stream key of a tensor: the seed and the name's CRC-32 through the same finaliser."""
    z = (int(seed) * _GOLDEN + zlib.crc32(name.encode("utf-8")) * _MUL2 + _MUL1) & ((1 << 64) - 1)
    z = ((z ^ (z >> 30)) * _MUL1) & ((1 << 64) - 1)
    z = ((z ^ (z >> 27)) * _MUL2) & ((1 << 64) - 1)
    return z ^ (z >> 31)


def standard_normal(key: int, begin: int, count: int, device: torch.device) -> torch.Tensor:
    """Elements begin .. begin+count of the stream `key`, fp32, the same bits on every device."""
    index = torch.arange(begin, begin + count, dtype=torch.int64, device=device)
    total = torch.zeros(count, dtype=torch.int64, device=device)
    for j in range(3):
        word = _finalise((index * 3 + (j + 1)) * _signed(_GOLDEN) + _signed(key))
        total += word & 0xFFFF
        for field in (1, 2, 3):
            total += _shift_right(word, 16 * field) & 0xFFFF
    return (total * 2 - 12 * 65535).to(torch.float32) * (1.0 / 131072.0)


def draw(spec: WeightSpec, seed: int, name: str, device: torch.device) -> torch.Tensor:
    """fp32 values of one tensor, computed on `device`; the bits do not depend on the device."""
    kind, std = spec.init
    if spec.role == "int_table":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    if kind not in ("normal", "one_plus_normal"):
        raise ValueError(f"unknown init {kind!r} for {name}")
    n = 1
    for s in spec.shape:
        n *= int(s)
    key = tensor_key(seed, name)
    out = torch.empty(n, dtype=torch.float32, device=device)
    for begin in range(0, n, _CHUNK):
        count = min(_CHUNK, n - begin)
        x = standard_normal(key, begin, count, device) * float(std)
        if kind == "one_plus_normal":
            x += 1.0
        out[begin:begin + count] = x
    return out.reshape(tuple(spec.shape))


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
    """Bind random weights to `model` in memory: the values a folder written by `write_random_model`
    with the same seed and storage dtype holds.  draw_on_device only says where the arithmetic runs
    (a large model is filled in seconds on the GPU)."""
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
