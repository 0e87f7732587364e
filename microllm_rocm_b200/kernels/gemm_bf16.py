"""bf16 x bf16 -> fp32-accumulated products for the serving path."""
from __future__ import annotations

from typing import Optional

import torch


def linear_bf16(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype,
                out: Optional[torch.Tensor]) -> torch.Tensor:
    from .build import LaunchCounter
    LaunchCounter.library += 1
    # Library product: cuBLASLt, bf16 operands, fp32 accumulate, output written in out_dtype.
    if out_dtype == torch.bfloat16:
        y = torch.mm(x, weight.t()) if out is None else torch.mm(x, weight.t(), out=out)
    else:
        y = torch.mm(x, weight.t(), out_dtype=torch.float32)
        if out is not None:
            out.copy_(y)
            y = out
    if bias is not None:
        y += bias.to(y.dtype)
    return y
