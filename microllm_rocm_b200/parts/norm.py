"""RMSNorm: y = x * (1 / sqrt(mean(x^2) + eps)) * w, all in fp32
(reference: src/ops/ops.cpp:684-699; fused with the residual add at :702-740)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from .base import Norm, Runtime, WeightSpec, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, params: dict, rt: Runtime):
        self.prefix = params.get("prefix", "")
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.rt = rt
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"weight": WeightSpec((self.size,), role="vector", init=("one_plus_normal", 0.1))}

    def bind(self, tensors):
        self.weight = tensors["weight"]

    def replay_key(self):
        return ("rmsnorm", self.size, self.eps)

    def own_tensors(self):
        return [self.weight]

    def forward(self, x, out, rows=None):
        ops.rmsnorm(x, self.weight, self.eps, out, rows=rows)

    def add_forward(self, residual, delta, out):
        ops.add_rmsnorm(residual, delta, self.weight, self.eps, out)
