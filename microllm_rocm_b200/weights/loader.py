"""Bind checkpoint tensors to a model's parts by name.

The model says which tensors it expects (full name -> shape and role); the file says which
it has.  Every disagreement -- missing, unexpected, wrong shape, unusable dtype -- is
collected and raised as ONE error before a single byte is copied, and nothing is bound
unless all is well: the reference's strict, atomic load with its
loaded/missing/unexpected/incompatible report (src/model/model.cpp:1679-1778; header
pre-flight before any payload is read :1838-1847).

Dtype policy on the device: matrices and tables in the compute dtype (bf16 stays bf16 in
the serving path; the reference widens everything to fp32, model.cpp:1877-1905); vectors
(norm weights, biases) in fp32, whose arithmetic is fp32 either way -- a tensor stored in
32 bits stays so; integer tables become int32.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Tuple

import torch

from ..parts.base import Runtime, WeightSpec
from .safetensors import SafetensorsFile, open_model_files

_FLOATS = (torch.float32, torch.bfloat16, torch.float16, torch.float64)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


@dataclass
class LoadReport:
    loaded: List[str] = field(default_factory=list)
    missing: List[str] = field(default_factory=list)
    unexpected: List[str] = field(default_factory=list)
    wrong_shape: List[Tuple[str, Tuple[int, ...], Tuple[int, ...]]] = field(default_factory=list)  # name, want, got
    wrong_dtype: List[Tuple[str, str]] = field(default_factory=list)
    ignored: List[str] = field(default_factory=list)

    @property
    def ok(self) -> bool:
        return not (self.missing or self.unexpected or self.wrong_shape or self.wrong_dtype)

    def message(self) -> str:
        lines = []
        if self.missing:
            lines.append(f"missing tensors ({len(self.missing)}): " + ", ".join(sorted(self.missing)))
        if self.unexpected:
            lines.append(f"unexpected tensors ({len(self.unexpected)}): " + ", ".join(sorted(self.unexpected)))
        if self.wrong_shape:
            lines.append(f"wrong shapes ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} expected {list(w)} got {list(g)}" for n, w, g in sorted(self.wrong_shape)))
        if self.wrong_dtype:
            lines.append(f"unusable dtypes ({len(self.wrong_dtype)}): " + ", ".join(
                f"{n} is {d}" for n, d in sorted(self.wrong_dtype)))
        return "; ".join(lines)


class WeightLoadError(ValueError):
    def __init__(self, report: LoadReport, where: str = ""):
        self.report = report
        super().__init__(f"weights do not fit the model{' (' + where + ')' if where else ''}: {report.message()}")


def target_dtype(role: str, rt: Runtime) -> torch.dtype:
    if role in ("matrix", "table"):
        return rt.dtype
    if role == "vector":
        return torch.float32
    if role == "int_table":
        return torch.int32
    raise ValueError(f"unknown tensor role {role!r}")


def check_names(expected: Dict[str, WeightSpec], available: Dict[str, Tuple[Tuple[int, ...], torch.dtype]],
                tolerated: List[str] = ()) -> LoadReport:
    """Compare what the model expects with what a checkpoint offers (name -> (shape, dtype))."""
    report = LoadReport()
    for name, spec in expected.items():
        if name not in available:
            report.missing.append(name)
            continue
        shape, dtype = available[name]
        if tuple(shape) != tuple(spec.shape):
            report.wrong_shape.append((name, tuple(spec.shape), tuple(shape)))
        elif spec.role == "int_table" and dtype not in _INTS:
            report.wrong_dtype.append((name, f"{dtype}, an integer table is expected"))
        elif spec.role != "int_table" and dtype not in _FLOATS:
            report.wrong_dtype.append((name, f"{dtype}, a floating-point tensor is expected"))
        else:
            report.loaded.append(name)
    for name in available:
        if name not in expected:
            (report.ignored if name in tolerated else report.unexpected).append(name)
    return report


def load_weights(model, folder_or_file: str, strict: bool = True) -> LoadReport:
    """Read the safetensors of a model folder into `model` (a parts.Model).  With
    strict=False unexpected tensors are reported but tolerated; anything missing or
    misshapen is always an error, since a model with holes cannot run."""
    files = open_model_files(folder_or_file)
    where: Dict[str, SafetensorsFile] = {}
    duplicates = []
    for f in files:
        for name in f.names():
            if name in where:
                duplicates.append(name)
            where[name] = f
    expected = model.expected_tensors()
    available = {n: (f.infos[n].shape, f.infos[n].torch_dtype) for n, f in where.items()}
    report = check_names(expected, available, model.tolerated_extra_tensors())
    if duplicates:
        report.unexpected.extend(f"{n} (in more than one shard)" for n in duplicates)
    if not strict and not (report.missing or report.wrong_shape or report.wrong_dtype or duplicates):
        report.ignored.extend(report.unexpected)
        report.unexpected = []
    if not report.ok:
        raise WeightLoadError(report, folder_or_file)
    rt: Runtime = model.rt
    tensors: Dict[str, torch.Tensor] = {}
    for name, spec in expected.items():
        src = where[name].tensor(name)
        tensors[name] = src.to(device=rt.device, dtype=target_dtype(spec.role, rt), non_blocking=False).contiguous()
    model.bind(tensors)
    return report
