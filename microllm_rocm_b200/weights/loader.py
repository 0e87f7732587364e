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

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

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
    load_ms: float = 0.0              # from the first byte staged to the last copy finished
    bytes_read: int = 0               # payload bytes taken from the file(s)

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
    started = time.perf_counter()
    destinations, pieces = model.placements()
    tensors: Dict[str, torch.Tensor] = {
        name: torch.empty(spec.shape, dtype=target_dtype(spec.role, rt), device=rt.device) for name, spec in destinations.items()}
    stream = _Stager(rt.device) if rt.device.type == "cuda" else None
    for name in expected:
        dest, row = pieces[name]
        src = where[name].tensor(name)
        target = tensors[dest]
        rows = src.shape[0] if src.dim() else 1
        into = target[row:row + rows] if target.dim() else target
        if tuple(into.shape) != tuple(src.shape):
            raise ValueError(f"tensor {name!r} of shape {list(src.shape)} does not fit rows {row}.. of {dest!r} {list(target.shape)}")
        if stream is not None:
            stream.copy(src, into)
        else:
            into.copy_(src)
        report.bytes_read += src.numel() * src.element_size()
    if stream is not None:
        stream.finish()
    report.load_ms = (time.perf_counter() - started) * 1e3
    model.bind(tensors)
    return report


class _Stager:
    """File -> device in bounded pieces: mapped file -> pinned host buffer (a ring of them, so that the next piece
    is staged while the last one travels) -> asynchronous copy, straight into the destination's rows when the
    file holds the destination's dtype, through a device buffer and a cast there when it does not.  The reference
    streams in the same manner (bounded staging, conversion on the device: src/model/model.cpp:1786-1908)."""

    def __init__(self, device: torch.device, piece_bytes: int = 32 << 20, buffers: int = 3):
        self.device, self.piece_bytes = device, piece_bytes
        self.pinned = [torch.empty(piece_bytes, dtype=torch.uint8, pin_memory=True) for _ in range(buffers)]
        self.events: List[Optional[torch.cuda.Event]] = [None] * buffers
        self.cast_buffer: Optional[torch.Tensor] = None
        self.next = 0

    def copy(self, src: torch.Tensor, into: torch.Tensor) -> None:
        """src: CPU tensor (a view of the mapped file); into: contiguous device tensor of the same shape."""
        if not into.is_contiguous():
            raise ValueError("the destination rows must be contiguous")
        n = src.numel()
        if n == 0:
            return
        flat_src = src.reshape(-1)
        flat_dst = into.view(-1) if into.dim() else into.reshape(1)
        same = src.dtype == into.dtype
        item = src.element_size()
        per_piece = max(1, self.piece_bytes // item)
        if not same and (self.cast_buffer is None or self.cast_buffer.numel() < self.piece_bytes):
            self.cast_buffer = torch.empty(self.piece_bytes, dtype=torch.uint8, device=self.device)
        for begin in range(0, n, per_piece):
            count = min(per_piece, n - begin)
            i = self.next
            self.next = (i + 1) % len(self.pinned)
            if self.events[i] is not None:
                self.events[i].synchronize()              # the copy that last read this buffer has run
            host = self.pinned[i][:count * item].view(src.dtype)
            host.copy_(flat_src[begin:begin + count])     # page cache -> pinned memory
            if same:
                flat_dst[begin:begin + count].copy_(host, non_blocking=True)
            else:
                staged = self.cast_buffer[:count * item].view(src.dtype)
                staged.copy_(host, non_blocking=True)
                flat_dst[begin:begin + count].copy_(staged)      # the cast, on the device, in stream order
            event = self.events[i] or torch.cuda.Event()
            event.record()
            self.events[i] = event

    def finish(self) -> None:
        torch.cuda.synchronize(self.device)
