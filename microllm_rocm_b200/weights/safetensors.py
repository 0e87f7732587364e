"""safetensors container: `u64 LE header length`, JSON header, payload.

Reader and writer with the checks the reference's reader makes
(src/io/safetensors.cpp:438-526): bounded header, known dtypes, every tensor's byte
range equal to shape x dtype size, ranges that tile the payload with no hole or overlap
and end at the end of the file, duplicate header keys rejected, `__metadata__` skipped.
The file is memory-mapped; tensors are views until they are copied to the device.
Sharded checkpoints through `model.safetensors.index.json` (`weight_map`, relative
paths that stay inside the folder: safetensors.cpp:635-670) are accepted too.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import torch

MAX_HEADER_BYTES = 256 << 20      # safetensors.cpp: header bound

_DTYPES = {
    "F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int          # offsets into the payload
    end: int
    file: str

    @property
    def torch_dtype(self) -> torch.dtype:
        return _DTYPES[self.dtype][0]


def _reject_duplicates(pairs):
    out = {}
    for k, v in pairs:
        if k in out:
            raise SafetensorsError(f"duplicate key {k!r} in safetensors header")
        out[k] = v
    return out


def _numel(shape: Iterable[int]) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


def inspect_file(path: str) -> Tuple[Dict[str, TensorInfo], int]:
    """Parse and validate the header; returns (infos by name, payload start offset)."""
    size = os.path.getsize(path)
    if size < 8:
        raise SafetensorsError(f"{path}: shorter than a safetensors header")
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        if hlen <= 0 or hlen > MAX_HEADER_BYTES or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} is invalid for a file of {size} bytes")
        raw = f.read(hlen)
    try:
        header = json.loads(raw.decode("utf-8"), object_pairs_hook=_reject_duplicates)
    except (UnicodeDecodeError, json.JSONDecodeError) as e:
        raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from None
    if not isinstance(header, dict):
        raise SafetensorsError(f"{path}: header must be a JSON object")
    payload = size - 8 - hlen
    infos: Dict[str, TensorInfo] = {}
    for name, d in header.items():
        if name == "__metadata__":
            continue
        try:
            dtype, shape, (b, e) = d["dtype"], tuple(int(s) for s in d["shape"]), d["data_offsets"]
        except (KeyError, TypeError, ValueError):
            raise SafetensorsError(f"{path}: entry {name!r} is malformed") from None
        if dtype not in _DTYPES:
            raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dtype!r}")
        if any(s < 0 for s in shape) or not (0 <= b <= e <= payload):
            raise SafetensorsError(f"{path}: tensor {name!r} has an invalid shape or byte range")
        if e - b != _numel(shape) * _DTYPES[dtype][1]:
            raise SafetensorsError(f"{path}: tensor {name!r}: {e - b} bytes do not match shape "
                                   f"{list(shape)} of {dtype}")
        infos[name] = TensorInfo(name, dtype, shape, int(b), int(e), path)
    cursor = 0
    for info in sorted(infos.values(), key=lambda i: (i.begin, i.end)):
        if info.begin != cursor:
            what = "a hole before" if info.begin > cursor else "an overlap at"
            raise SafetensorsError(f"{path}: payload has {what} tensor {info.name!r}")
        cursor = info.end
    if cursor != payload:
        raise SafetensorsError(f"{path}: payload is {payload} bytes but tensors cover {cursor}")
    return infos, 8 + hlen


class SafetensorsFile:
    """A memory-mapped safetensors file; `tensor(name)` is a CPU view, not a copy."""

    def __init__(self, path: str):
        self.path = path
        self.infos, self._start = inspect_file(path)
        self._fh = open(path, "rb")
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if os.path.getsize(path) else None

    def names(self) -> List[str]:
        return list(self.infos)

    def tensor(self, name: str) -> torch.Tensor:
        info = self.infos[name]
        n = _numel(info.shape)
        if n == 0:
            return torch.empty(info.shape, dtype=info.torch_dtype)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")       # the mapping is read-only; we never write to it
            flat = torch.frombuffer(self._map, dtype=info.torch_dtype, count=n,
                                    offset=self._start + info.begin)
        return flat.reshape(info.shape)

    def close(self) -> None:
        # views may still reference the mapping; let the garbage collector unmap it
        self._fh.close()


def open_model_files(folder_or_file: str) -> List[SafetensorsFile]:
    """The safetensors file(s) of a model folder: model.safetensors, or the shards that
    model.safetensors.index.json lists."""
    if os.path.isfile(folder_or_file):
        return [SafetensorsFile(folder_or_file)]
    single = os.path.join(folder_or_file, "model.safetensors")
    if os.path.isfile(single):
        return [SafetensorsFile(single)]
    index = os.path.join(folder_or_file, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            weight_map = json.load(f).get("weight_map")
        if not isinstance(weight_map, dict) or not weight_map:
            raise SafetensorsError(f"{index}: weight_map is missing or empty")
        shards = []
        for rel in sorted(set(weight_map.values())):
            if os.path.isabs(rel) or ".." in rel.replace("\\", "/").split("/"):
                raise SafetensorsError(f"{index}: shard path {rel!r} leaves the model folder")
            shards.append(SafetensorsFile(os.path.join(folder_or_file, rel)))
        for name, rel in weight_map.items():
            if not any(s.path.endswith(rel) and name in s.infos for s in shards):
                raise SafetensorsError(f"{index}: tensor {name!r} is not in shard {rel!r}")
        return shards
    raise FileNotFoundError(f"no model.safetensors (or index) in {folder_or_file}")


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: Dict[str, str] = None) -> None:
    """Write tensors (CPU or device) in the order given; the file appears atomically."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    cursor = 0
    for name, t in tensors.items():
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [cursor, cursor + nbytes]}
        cursor += nbytes
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * ((8 - len(raw) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for t in tensors.values():
            c = t.detach().contiguous().cpu()
            if c.numel():
                f.write(c.view(torch.uint8).reshape(-1).numpy().tobytes() if c.dim() else
                        c.reshape(1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)
