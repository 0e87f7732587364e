"""Token embedding (gather of table rows into the fp32 residual stream) and the LM head
(product of selected, normalised rows with the head matrix, or with the embedding table
when the two are tied).  Reference: embedding src/ops/ops.cpp:581-618; tied head as a
product with the transposed table, no copy, src/model/model.cpp:1122-1125."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from ..kernels.linear import linear
from .base import Part, Runtime, WeightSpec, register_embedding, register_head


@register_embedding("token_embedding")
class TokenEmbedding(Part):
    def __init__(self, params: dict, rt: Runtime):
        self.name = params["name"]
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.rt = rt
        self.table: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.name: WeightSpec((self.vocab, self.hidden), role="table")}

    def bind(self, tensors):
        self.table = tensors[self.name]

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        out = torch.empty((token_ids.shape[0], self.hidden), dtype=torch.float32, device=token_ids.device)
        ops.embed_gather(self.table, token_ids, out)
        return out


@register_head("lm_head")
class LMHead(Part):
    def __init__(self, params: dict, rt: Runtime):
        self.name = params["name"]
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.tied_to = params.get("tied_to")
        self.rt = rt
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        if self.tied_to is not None:
            return {}
        return {self.name: WeightSpec((self.vocab, self.hidden), role="matrix")}

    def bind(self, tensors):
        self.weight = tensors[self.tied_to if self.tied_to is not None else self.name]

    def kernel_sources(self):
        if self.rt.is_fp32:
            return []
        from ..kernels import gemm_bf16
        return gemm_bf16.sources(engine_only=True)

    def forward(self, rows: torch.Tensor, error_flag: Optional[torch.Tensor] = None) -> torch.Tensor:
        """rows [R, H] in the compute dtype -> logits [R, V] fp32.  `error_flag`: the step's device flag."""
        logits = linear(rows, self.weight, None, torch.float32, partials_ok=True, error_flag=error_flag)
        if logits.dim() == 3:
            # a weight-streaming kernel: with this many output rows it does not split K, so the one
            # partial result is the product itself
            if logits.shape[0] != 1:        # a small vocabulary with a long K: add the partial results up
                total = torch.zeros(logits.shape[1:], dtype=torch.float32, device=logits.device)
                ops.add_inplace(total, logits)
                logits = total
            else:
                logits = logits[0]
        return logits
