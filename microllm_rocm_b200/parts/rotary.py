"""Rotary position encoding as a table of inverse frequencies.

inv_freq[i] = theta^(-2 i / rotary_dim), evaluated in fp32 exactly as the reference does
per element (src/ops/ops.cpp:861-864: `std::pow(base, -2.0F * float(pair) / float(head_width))`).
The reference recomputes it inside every kernel call; here it is computed once.  Layout
'split_half' pairs element i with i + rotary_dim/2 (the reference's SplitHalf,
src/model/config.h:9), 'interleaved' pairs 2i with 2i+1.  `rotary_dim` smaller than the
head size leaves the remaining elements untouched.  Optional `scale` divides positions'
frequencies (linear scaling); it defaults to 1.
"""
from __future__ import annotations

import numpy as np
import torch

from .base import PositionEncoding, RotaryTable, Runtime, register_position_encoding


def inverse_frequencies(theta: float, rotary_dim: int, scale: float = 1.0) -> np.ndarray:
    i = np.arange(rotary_dim // 2, dtype=np.float32)
    exponent = (np.float32(-2.0) * i) / np.float32(rotary_dim)
    inv = np.power(np.float32(theta), exponent, dtype=np.float32)
    if scale != 1.0:
        inv = (inv / np.float32(scale)).astype(np.float32)
    return inv


@register_position_encoding("rotary")
class RotaryEmbedding(PositionEncoding):
    def __init__(self, params: dict, rt: Runtime):
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        self.theta = float(params["theta"])
        self.layout = params.get("layout", "split_half")
        self.scale = float(params.get("scale", 1.0))
        if self.layout not in ("split_half", "interleaved"):
            raise ValueError(f"rotary layout {self.layout!r} is not one of split_half, interleaved")
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError("rotary_dim must be even and at most head_dim")
        if not self.theta > 0:
            raise ValueError("rotary theta must be positive")
        inv = inverse_frequencies(self.theta, self.rotary_dim, self.scale)
        self._table = RotaryTable(torch.from_numpy(inv).to(rt.device), self.rotary_dim,
                                  self.layout == "interleaved")

    def rotary_table(self, head_dim: int):
        if head_dim != self.head_dim:
            raise ValueError(f"rotary table was built for head_dim {self.head_dim}, asked for {head_dim}")
        return self._table


@register_position_encoding("none")
class NoPositionEncoding(PositionEncoding):
    def __init__(self, params: dict, rt: Runtime):
        pass
