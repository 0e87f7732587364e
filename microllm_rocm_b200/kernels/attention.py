"""Choice of the attention kernel for a step.

fp32: always the plain kernel (fixed summation order, bit-stable across ways of cutting).
bf16: the tensor-core kernels when the head size is a multiple of 32 and the page size a
multiple of 16; the plain kernel otherwise.  A step whose sequences all bring one token runs
the decode shape of `attention_mma.cu` (keys split over a thread-block cluster that merges
through distributed shared memory).  In any other step every sequence that brings two tokens or
more goes to the tcgen05 kernel (`attention_tc.cu`: 128 query rows per CTA, scores and output in
tensor memory; head sizes 64 and 128), every sequence that brings exactly one token (a decoded
token beside prompt portions) to the decode shape again, through a list of those sequences.  Head
sizes the tcgen05 kernel does not take go to the prefill shape of `attention_mma.cu` with its
16-row tiles.  The launches write disjoint rows of the output.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import build, ops
from .build import KernelError
from .device import DEFAULT_SM_COUNT, sm_count

MAX_HEAD_DIM = 256
MIN_KEY_TILES_PER_SPLIT = 4         # one 16-key tile per warp at least
DECODE_SPLITS = (16, 8, 4, 2)       # cluster sizes tried, largest first
WIDE_CLUSTER_CTAS = 48              # measured: one sequence of two kv heads gains 3 % from clusters of 16, eight sequences lose 10 %

# Which decode kernel takes heads of 128: None = by the step's shape (`decode_ring_pays`); True / False = always /
# never.  Tests set it to run both kernels on the same inputs.
DECODE_RING = None
RING_MIN_KEYS_PER_CTA = 1024        # measured: 16 stages of 64 keys per CTA and the ring wins by 7-8 %, 8 stages and it loses 12 %
# Measured in whole decode steps at context 8,192 (8 layers of the 14B / 7B shapes), when the products around the
# attention were still the few-token mma.sync kernels: with 8 tokens the ring cost 2.64 against 2.01 ms / 2.08
# against 1.50 ms although the kernel alone is 8 % faster; with 16 tokens (tcgen05 streaming products around it)
# it won, 2.03 against 2.42 / 1.35 against 1.52 ms.  The mma.sync products' CTAs take up to 160 KB of shared memory:
# beside two ring CTAs (113 KB each) they cannot start early.  Since the wide models' few-token products went to
# the streaming kernel too, the ring wins there at 8 tokens as well (14B: 1.85 -> 1.67 ms, 7B: 1.28 -> 1.19 ms).
# So the caller says which products surround the attention (`beside_mma_products`).
CONCURRENT_ATTENTION = True         # the two attention launches of a mixed step side by side (tests may switch it off)
TC_HEAD_DIMS = (64, 128)
TC_KEYS_PER_TILE = 128
TC_ROWS_PER_TILE = 128
# Measured with one sequence of 2 to 47 new tokens at contexts of 64 to 4,096 keys (heads 12/2 and 28/4 of 128): the
# tcgen05 kernel takes 7.4 to 48 us where the mma.sync kernel's 16-row tiles take 8.4 to 230: it wins everywhere.
TC_MIN_NEW_TOKENS = 2

ops.register_signatures("attention_tc.cu", {
    "mlb_fa_tc_supported": [c_int, c_float],
    "mlb_paged_attention_tc": [c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p,
                               c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
})
ops.register_signatures("attention_mma.cu", {
    "mlb_paged_attention_mma": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p],
})


def check_head_dim(d: int) -> None:
    """Refuse a head size the kernels cannot take, before any weight is loaded."""
    if d <= 0 or d % 2 or d > MAX_HEAD_DIM:
        raise KernelError(f"head_dim {d} is not supported: it must be even and at most {MAX_HEAD_DIM}")


def mma_supported(head_dim: int, page_size: int) -> bool:
    return head_dim % 32 == 0 and 32 <= head_dim <= MAX_HEAD_DIM and page_size % 16 == 0


def mma_sources(head_dim: int):
    return [("attention_mma.cu", {"HEAD_DIM": head_dim})] if head_dim % 32 == 0 and 32 <= head_dim <= MAX_HEAD_DIM else []


def tc_supported(head_dim: int, page_size: int, scale: float) -> bool:
    return (head_dim in TC_HEAD_DIMS and page_size % 8 == 0 and TC_KEYS_PER_TILE % page_size == 0
            and TC_KEYS_PER_TILE // page_size <= 16 and scale > 0.0)


def tc_sources(head_dim: int):
    return [("attention_tc.cu", {"HEAD_DIM": head_dim})] if head_dim in TC_HEAD_DIMS else []


def decode_splits(items: int, max_seq_len: int, sms: int = DEFAULT_SM_COUNT) -> int:
    """How many CTAs (one thread-block cluster) share the keys of one (sequence, kv head) in a decode step:
    as many as still fit the GPU's `sms` multiprocessors in one wave (two CTAs per SM) and leave every warp a
    key tile."""
    key_tiles = max(1, -(-max_seq_len // 16))
    items = max(1, items)
    for cand in DECODE_SPLITS:
        if cand > 8 and items * cand > WIDE_CLUSTER_CTAS:
            continue          # clusters of 16 pay only while the whole grid is a handful of (eight-warp) CTAs
        if items * cand <= sms * 2 and key_tiles >= cand * MIN_KEY_TILES_PER_SPLIT:
            return cand
    return 1


def decode_ring_pays(items: int, splits: int, max_seq_len: int, sms: int = DEFAULT_SM_COUNT,
                     beside_mma_products: bool = False) -> bool:
    """Whether a decode step should bring its keys through the shared-memory ring (TMA, a copying warp) instead of
    straight into registers: when every multiprocessor has a CTA, each CTA streams a thousand keys or more, and
    the products around the attention are not the few-token mma.sync kernels.  Below that the ring's set-up and
    its extra hand-offs cost more than the deeper prefetch brings; beside those kernels its shared memory keeps
    the next one from starting early."""
    return (items * splits >= sms and max_seq_len // max(1, splits) >= RING_MIN_KEYS_PER_CTA and splits <= 8
            and not beside_mma_products)


def decode_plan_stale(ctx, max_seq_len: int, sms: int = DEFAULT_SM_COUNT) -> bool:
    """Whether a decode step planned for `ctx` (its plans are kept in ctx.extras, and frozen into a captured
    graph) would be cut differently at this context length: a step captured at a short context has one CTA
    per (sequence, kv head) and must not serve a context of thousands that way."""
    for key, plan in ctx.extras.items():
        if isinstance(key, tuple) and key and key[0] == "attention_mma" and plan[2] == 1:
            splits = decode_splits(plan[1] * key[2], max_seq_len, sms)
            beside = bool(key[4]) if len(key) > 4 else False
            if splits != plan[3] or (len(plan) > 9 and decode_ring_pays(plan[1] * key[2], splits, max_seq_len, sms, beside) != plan[9]):
                return True
    return False


def forget_plans(ctx) -> None:
    for key in [k for k in ctx.extras if isinstance(k, tuple) and k and k[0] == "attention_mma"]:
        del ctx.extras[key]


def _plan(ctx, group: int, num_kv_heads: int, use_tc: bool, beside_mma_products: bool = False):
    """Work lists and split choice of a step, shared by every layer with the same group size."""
    key = ("attention_mma", group, num_kv_heads, use_tc, bool(beside_mma_products))
    plan = ctx.extras.get(key)
    if plan is not None:
        return plan
    starts, A = ctx.seq_starts_host, ctx.num_seqs
    decode = ctx.max_new_tokens == 1
    work, tc_work, listed = [], [], []
    tiles_per_token = -(-group // 16)
    for a in range(A):
        n_new = starts[a + 1] - starts[a]
        if use_tc and not decode and n_new >= TC_MIN_NEW_TOKENS:
            pos0 = ctx.seq_pos0_host[a]
            for tile in range(-(-n_new // TC_ROWS_PER_TILE)):
                last_pos = pos0 + min(n_new, (tile + 1) * TC_ROWS_PER_TILE) - 1
                tc_work.append((last_pos // TC_KEYS_PER_TILE, a, tile))
            continue
        if not decode and n_new == 1:
            listed.append(a)          # a decoded token beside prompt portions: the decode shape, with its key split
            continue
        tiles = -(-n_new * group // 16)
        work += [(a, first) for first in range(0, tiles, 1 if decode else 4)]
    if not decode:
        # causal work grows with the row tile: start the long ones first so that the tail is short
        work.sort(key=lambda item: -item[1])
        tc_work.sort(key=lambda item: -item[0])
    device = ctx.positions.device
    sms = sm_count(device)
    # (through pinned memory: a copy from pageable memory would first wait for the whole stream, and with it for the
    # step before this one, which may still be running)
    # the three lists travel as one array (the kernels read them int by int: no alignment beyond 4 bytes is needed)
    flat_work = [x for item in work for x in item]
    flat_tc = [x for _, a, t in tc_work for x in (a, t)]
    lists = ops.upload(flat_work + flat_tc + listed, "int32", device)
    work_dev = lists[:len(flat_work)]
    tc_dev = lists[len(flat_work):len(flat_work) + len(flat_tc)]
    splits = decode_splits(len(work) * num_kv_heads, ctx.max_seq_len, sms) if decode else 1
    ring = decode and decode_ring_pays(len(work) * num_kv_heads, splits, ctx.max_seq_len, sms, beside_mma_products)
    listed_dev, listed_splits = None, 1
    if listed:
        listed_dev = lists[len(flat_work) + len(flat_tc):]
        longest = max(ctx.seq_pos0_host[a] for a in listed) + 1
        listed_splits = decode_splits(len(listed) * tiles_per_token * num_kv_heads, longest, sms)
        ring = decode_ring_pays(len(listed) * tiles_per_token * num_kv_heads, listed_splits, longest, sms, beside_mma_products)
    plan = (work_dev, len(work), 1 if decode else 0, splits, tc_dev, len(tc_work), listed_dev, len(listed) * tiles_per_token,
            listed_splits, ring)
    ctx.extras[key] = plan
    return plan


def paged_attention(q: torch.Tensor, pages: torch.Tensor, out: torch.Tensor, ctx, block_table: torch.Tensor,
                    num_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: Optional[int],
                    beside_mma_products: bool = False) -> None:
    """`beside_mma_products`: the projections around this attention run on the few-token mma.sync kernels in this
    step (a choice of the caller's products; it decides which decode kernel suits, see decode_ring_pays)."""
    page_size = pages.shape[3]
    if q.dtype != torch.bfloat16 or not mma_supported(head_dim, page_size):
        ops.paged_attention_plain(q, pages, out, ctx.positions, ctx.token_seq, block_table, num_heads, num_kv_heads,
                                  head_dim, scale, window, ctx.error_flag)
        return
    if pages.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("paged_attention: the tensor-core kernel wants bf16 queries, pages and output")
    use_tc = tc_supported(head_dim, page_size, scale) and q.is_contiguous() and out.is_contiguous()
    work, num_work, mode, splits, tc_work, num_tc, listed, num_listed, listed_splits, ring = _plan(
        ctx, num_heads // num_kv_heads, num_kv_heads, use_tc, beside_mma_products)
    ring_bits = 4 if (ring if DECODE_RING is None else DECODE_RING) else 8
    side = None
    if num_tc:
        # Prompt portions and the decoded tokens beside them are different sequences: their two launches write
        # disjoint rows and read nothing of each other's.  The prompt portions' kernel goes to the device's second
        # stream, so that both run at once (it leaves a quarter of the SMs idle at the benchmark's sizes).
        stream = ops._stream()
        if (num_work or num_listed) and CONCURRENT_ATTENTION:
            side = ops.side_stream()
            ops.fork(side)
            stream = side
        T = ops.lib("attention_tc.cu", {"HEAD_DIM": head_dim})
        build.check(T, T.mlb_paged_attention_tc(
            q.data_ptr(), q.stride(0), pages.data_ptr(), out.data_ptr(), out.stride(0), q.shape[0], ctx.seq_starts.data_ptr(),
            ctx.seq_pos0.data_ptr(), block_table.data_ptr(), tc_work.data_ptr(), num_tc, block_table.shape[1],
            pages.shape[0], page_size, num_heads, num_kv_heads, int(window or 0), float(scale), ops._ptr(ctx.error_flag),
            stream))
    if not num_work and not num_listed:
        return
    L = ops.lib("attention_mma.cu", {"HEAD_DIM": head_dim})
    if num_listed:
        # decoded tokens beside prompt portions: the decode shape for the listed sequences (mode 2)
        build.check(L, L.mlb_paged_attention_mma(
            q.data_ptr(), pages.data_ptr(), out.data_ptr(), ctx.seq_starts.data_ptr(), ctx.seq_pos0.data_ptr(), block_table.data_ptr(),
            listed.data_ptr(), num_listed, block_table.shape[1], pages.shape[0], page_size, num_heads, num_kv_heads,
            int(window or 0), float(scale), 2 + ring_bits, listed_splits, ops._ptr(ctx.error_flag), ops._stream()))
    if num_work:
        build.check(L, L.mlb_paged_attention_mma(
            q.data_ptr(), pages.data_ptr(), out.data_ptr(), ctx.seq_starts.data_ptr(), ctx.seq_pos0.data_ptr(), block_table.data_ptr(), work.data_ptr(), num_work,
            block_table.shape[1], pages.shape[0], page_size, num_heads, num_kv_heads, int(window or 0), float(scale),
            mode + (ring_bits if mode else 0), splits, ops._ptr(ctx.error_flag), ops._stream()))
    if side is not None:
        ops.join(side)
