"""Choice of the attention kernel for a step.

fp32: always the plain kernel (fixed summation order, bit-stable across ways of cutting).
bf16: the plain kernel too until the tensor-core kernels take a case over (see
`FAST_KERNELS`); every fast kernel is tested against the plain one.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops
from .build import KernelError

MAX_HEAD_DIM = 256


def check_head_dim(d: int) -> None:
    """Refuse a head size the kernels cannot take, before any weight is loaded."""
    if d <= 0 or d % 2 or d > MAX_HEAD_DIM:
        raise KernelError(f"head_dim {d} is not supported: it must be even and at most {MAX_HEAD_DIM}")


def paged_attention(q: torch.Tensor, pages: torch.Tensor, out: torch.Tensor, ctx, block_table: torch.Tensor,
                    num_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: Optional[int]) -> None:
    ops.paged_attention_plain(q, pages, out, ctx.positions, ctx.token_seq, block_table, num_heads, num_kv_heads,
                              head_dim, scale, window, ctx.error_flag)
