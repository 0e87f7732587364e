"""Choice of the attention kernel for a step.

fp32: always the plain kernel (fixed summation order, bit-stable across ways of cutting).
bf16: the tensor-core kernel (`attention_mma.cu`, compiled for the model's head size) when
the head size is a multiple of 32 and the page size a multiple of 16; the plain kernel
otherwise.  A step whose sequences all bring one token runs the decode shape (keys split
over CTAs, partial results in scratch memory, merged by the CTA that finishes last); any
other step runs the prefill shape.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_void_p
from typing import Optional

import torch

from . import build, ops
from .build import KernelError

MAX_HEAD_DIM = 256
SM_COUNT = 148
MAX_SPLITS = 64
MIN_KEY_TILES_PER_SPLIT = 4         # one 16-key tile per warp at least

ops.register_signatures("attention_mma.cu", {
    "mlb_paged_attention_mma": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                c_int, c_int, c_void_p, c_void_p],
})


def check_head_dim(d: int) -> None:
    """Refuse a head size the kernels cannot take, before any weight is loaded."""
    if d <= 0 or d % 2 or d > MAX_HEAD_DIM:
        raise KernelError(f"head_dim {d} is not supported: it must be even and at most {MAX_HEAD_DIM}")


def mma_supported(head_dim: int, page_size: int) -> bool:
    return head_dim % 32 == 0 and 32 <= head_dim <= MAX_HEAD_DIM and page_size % 16 == 0


def mma_sources(head_dim: int):
    return [("attention_mma.cu", {"HEAD_DIM": head_dim})] if head_dim % 32 == 0 and 32 <= head_dim <= MAX_HEAD_DIM else []


def _plan(ctx, group: int, num_kv_heads: int):
    """Work list and split choice of a step, shared by every layer with the same group size."""
    key = ("attention_mma", group, num_kv_heads)
    plan = ctx.extras.get(key)
    if plan is not None:
        return plan
    starts, A = ctx.seq_starts_host, ctx.num_seqs
    decode = ctx.max_new_tokens == 1
    work = []
    for a in range(A):
        tiles = -(-(starts[a + 1] - starts[a]) * group // 16)
        work += [(a, first) for first in range(0, tiles, 1 if decode else 4)]
    work_dev = torch.tensor(work, dtype=torch.int32).reshape(-1).to(ctx.positions.device, non_blocking=True)
    splits, long_loops = 1, 0
    if decode:
        # each CTA takes an even share of its own sequence's keys, so the launch shape chosen
        # here stays balanced while the sequences of a captured step grow
        key_tiles = max(1, -(-ctx.max_seq_len // 16))
        items = max(1, len(work) * num_kv_heads)

        def choose(resident_per_sm):
            return max(1, min(SM_COUNT * resident_per_sm // items, key_tiles // MIN_KEY_TILES_PER_SPLIT, MAX_SPLITS))

        splits = choose(3)                     # the lean kernel: three CTAs per SM, one wave
        if -(-key_tiles // splits) > 8:        # warps would walk more than two key tiles each:
            long_loops = 1                     # the prefetching kernel (two CTAs per SM) pays
            splits = choose(2)
    # one ticket per (work item, kv head): which split finished last; the kernel leaves them zero
    tickets = torch.zeros(len(work) * num_kv_heads, dtype=torch.int32, device=ctx.positions.device) if splits > 1 else None
    plan = (work_dev, len(work), 1 if decode else 0, splits, tickets, long_loops)
    ctx.extras[key] = plan
    return plan


def paged_attention(q: torch.Tensor, pages: torch.Tensor, out: torch.Tensor, ctx, block_table: torch.Tensor,
                    num_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: Optional[int]) -> None:
    page_size = pages.shape[3]
    if q.dtype != torch.bfloat16 or not mma_supported(head_dim, page_size):
        ops.paged_attention_plain(q, pages, out, ctx.positions, ctx.token_seq, block_table, num_heads, num_kv_heads,
                                  head_dim, scale, window, ctx.error_flag)
        return
    if pages.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("paged_attention: the tensor-core kernel wants bf16 queries, pages and output")
    T = q.shape[0]
    work, num_work, mode, splits, tickets, long_loops = _plan(ctx, num_heads // num_kv_heads, num_kv_heads)
    part_o = part_lse = None
    if splits > 1:
        part_o = torch.empty((T * num_heads, splits, head_dim), dtype=torch.float32, device=q.device)
        part_lse = torch.empty((T * num_heads, splits), dtype=torch.float32, device=q.device)
    L = ops.lib("attention_mma.cu", {"HEAD_DIM": head_dim})
    build.check(L, L.mlb_paged_attention_mma(
        q.data_ptr(), pages.data_ptr(), out.data_ptr(), ops._ptr(part_o), ops._ptr(part_lse), ops._ptr(tickets),
        ctx.seq_starts.data_ptr(), ctx.seq_pos0.data_ptr(), block_table.data_ptr(), work.data_ptr(), num_work,
        block_table.shape[1], pages.shape[0], page_size, num_heads, num_kv_heads, int(window or 0), float(scale),
        mode, splits, long_loops, ops._ptr(ctx.error_flag), ops._stream()))
