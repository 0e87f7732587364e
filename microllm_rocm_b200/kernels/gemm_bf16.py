"""bf16 x bf16 -> fp32-accumulated products of the serving path.

Who takes which product (`linear_bf16`, and the parts for their fused forms):
  up to 8 tokens      the weight-streaming mma.sync kernels (`gemv_bf16.cu`, `gemv_fused.cu`)
  9 to 128 tokens     the weight-streaming tcgen05 kernel (`gemm_stream.cu`): fp32 partial results for QKV, O,
                      down and the head; gate/up with its activation as the epilogue
  256 tokens and up   gate/up with its activation: the CTA-pair tcgen05 kernel (`gemm_tc2.cu`)
  everything else     the library product, cuBLASLt called through `gemm_lib.cu` (or through torch.mm when a
                      bias has to be added or cuBLASLt cannot be taken from the process)
Grid sizes and K splits follow the multiprocessor count of the device the operands live on.
"""
from __future__ import annotations

from ctypes import c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import build, ops
from .build import KernelError, LaunchCounter
from .device import DEFAULT_SM_COUNT, sm_count

ops.register_signatures("gemv_bf16.cu", {
    "mlb_gemv_bf16": [c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_int,
                      c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
})
ops.register_signatures("gemv_fused.cu", {
    "mlb_gemv_split": [c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                       c_int, c_void_p],
    "mlb_gemv_silu": [c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_void_p, c_longlong, c_int, c_int, c_int,
                      c_void_p],
    "mlb_gemv_qkv_rope": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                          c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                          c_void_p],
})
ops.register_signatures("gemm_lib.cu", {
    "mlb_lt_available": [],
    "mlb_lt_matmul": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int,
                      c_void_p, c_longlong, c_void_p],
})
ops.register_signatures("gemm_tc2.cu", {
    "mlb_gemm_pair": [c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_longlong, c_int, c_int,
                      c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
})
ops.register_signatures("gemm_stream.cu", {
    "mlb_gemm_stream_max_tokens": [],
    "mlb_gemm_stream_splits": [c_int, c_int],
    "mlb_gemm_stream": [c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                        c_int, c_void_p, c_void_p],
    "mlb_gemm_stream_silu": [c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_void_p, c_longlong, c_int, c_int,
                             c_int, c_int, c_void_p, c_void_p],
})

_error_flags = {}

LIBRARY_WORKSPACE_BYTES = 32 << 20
_workspaces = {}
_direct_ok = None


def sources(engine_only: bool = False):
    """The objects of this module; with engine_only just those that a model's step can reach."""
    return [("gemm_tc2.cu", {}), ("gemm_stream.cu", {}), ("gemv_bf16.cu", {}), ("gemv_fused.cu", {}), ("gemm_lib.cu", {})]


# ------------------------------------------------------------------------------ few tokens: weight streaming
GEMV_MAX_TOKENS = 16                  # what the mma.sync weight-streaming kernels can take
# ...and up to where the engine sends them: from 9 tokens on (a second 8-token column block per fragment) the
# tcgen05 streaming kernel is the faster one
GEMV_ROUTE_MAX_TOKENS = 8
GEMV_CTAS_PER_SM = 4                  # CTAs the one-warp-per-range kernel aims at
GEMV_MIN_K_PER_SPLIT = 256


def gemv_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    m, k = x.shape
    return (0 < m <= GEMV_MAX_TOKENS and k % 32 == 0 and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0
            and x.stride(1) == 1 and weight.stride(1) == 1 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def gemv_splits(n: int, k: int, sms: int = DEFAULT_SM_COUNT):
    """(splits, k_per_split): enough CTAs to fill the GPU, K ranges of whole 32-element chunks."""
    row_blocks = -(-n // 64)
    splits = max(1, min(-(-GEMV_CTAS_PER_SM * sms // row_blocks), k // GEMV_MIN_K_PER_SPLIT))
    k_per_split = -(-(-(-k // splits)) // 32) * 32
    while k_per_split * 2 * 16 > 160 * 1024:                 # the staged activations must fit shared memory
        k_per_split = -(-(k_per_split // 2) // 32) * 32
    return -(-k // k_per_split), k_per_split


def _empty(shape, dtype, device, alloc):
    return alloc(shape, dtype) if alloc is not None else torch.empty(shape, dtype=dtype, device=device)


def gemv_partials(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, alloc=None) -> torch.Tensor:
    """[S, M, N] fp32 partial results of x @ weight^T (+ bias, in partial 0); their sum over S,
    taken in order by the kernel that consumes them, is the product.  `alloc(shape, dtype)`: where the
    result comes from (a step's scratch; default: a new tensor)."""
    M, K = x.shape
    N = weight.shape[0]
    sms = sm_count(x.device)
    plan = gemv_split_plan(N, K, sms) if x.dtype == torch.bfloat16 and M >= GEMV_SPLIT_MIN_TOKENS else None
    if plan is not None:
        return gemv_split_partials(x, weight, bias, *plan, alloc=alloc)
    splits, k_per_split = gemv_splits(N, K, sms)
    partial = _empty((splits, M, N), torch.float32, x.device, alloc)
    L = ops.lib("gemv_bf16.cu")
    build.check(L, L.mlb_gemv_bf16(x.data_ptr(), x.stride(0), weight.data_ptr(), weight.stride(0), N, ops._ptr(bias),
                                   partial.data_ptr(), None, 0, 0, 0, M, N, K, splits, k_per_split, ops._stream()))
    return partial


GEMV_SILU_MAX_TOKENS = 8            # beyond one 8-token column block the fused gate/up kernel loses to partial sums + activation
GEMV_FUSED_MAX_K = 6144             # the activations of 16 tokens over the whole K must fit shared memory


# The mma.sync kernels stage the step's activations over their K range in shared memory (16 token rows).  Up to
# this many elements of K per CTA (96 KB) two of their CTAs share an SM, so that the next kernel's CTAs become
# resident, and fetch their first weights, while this kernel still runs; a wider product takes the SM for itself
# and loses that.  Then the tcgen05 streaming kernel, whose TMA-filled ring keeps more of the weight stream in
# flight than registers can, is the faster one at ANY token count.  Measured in whole decode steps of 1 and 8
# tokens: every product of the 7B and 14B shapes (K = 3,584 / 5,120: 112 / 160 KB staged) gains on the streaming
# kernel (8 layers: 1.36 -> 1.06 ms and 1.72 -> 1.45 ms), every product of the 1.5B shape (K = 1,536, and 2,987 per
# CTA for the down projection) loses there (1.235 -> 1.374 ms for all of them, 28 layers).
GEMV_MAX_STAGED_K = 3072


def gemv_staged_k(n: int, k: int, sms: int = DEFAULT_SM_COUNT) -> int:
    """Elements of K whose activations one CTA of the mma.sync kernels keeps in shared memory."""
    if k <= GEMV_FUSED_MAX_K:
        return k
    plan = gemv_split_plan(n, k, sms)
    return plan[1] if plan is not None else gemv_splits(n, k, sms)[1]


def gemv_preferred(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """The mma.sync weight-streaming kernels can take this product and are the faster way for it."""
    if not (x.shape[0] <= GEMV_ROUTE_MAX_TOKENS and gemv_supported(x, weight)):
        return False
    if gemv_staged_k(weight.shape[0], x.shape[1], sm_count(x.device)) <= GEMV_MAX_STAGED_K:
        return True
    return not stream_supported(x, weight)


def gemv_fused_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """The few-token kernels that finish their own epilogue (activation; rotation and cache store)."""
    return gemv_supported(x, weight) and x.shape[1] <= GEMV_FUSED_MAX_K and x.dtype == torch.bfloat16


GEMV_SPLIT_CTAS_PER_SM = 2              # eight-warp CTAs, two per SM
GEMV_SPLIT_MIN_TOKENS = 8               # measured: below this the one-warp-per-range kernel is the faster one (1.205 against 1.226 ms at batch 6)
GEMV_SPLIT_MAX_TILES_PER_SM = 4         # beyond this many 16-row tiles the one-warp-per-range kernel streams better


def gemv_split_plan(n: int, k: int, sms: int = DEFAULT_SM_COUNT):
    """(splits, k_per_cta) for the kernel that splits K inside the CTA, or None when the other kernel suits better."""
    tiles = -(-n // 16)
    if tiles > GEMV_SPLIT_MAX_TILES_PER_SM * sms:
        return None
    splits = max(1, min(GEMV_SPLIT_CTAS_PER_SM * sms // tiles, k // GEMV_MIN_K_PER_SPLIT))
    k_per_cta = -(-(-(-k // splits)) // 32) * 32
    while k_per_cta > GEMV_FUSED_MAX_K:
        splits += 1
        k_per_cta = -(-(-(-k // splits)) // 32) * 32
    return -(-k // k_per_cta), k_per_cta


def gemv_split_partials(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], splits: int,
                        k_per_cta: int, alloc=None) -> torch.Tensor:
    """[S, M, N] fp32 partial results from the kernel whose warps share a CTA's K range (few partials)."""
    M, K = x.shape
    N = weight.shape[0]
    partial = _empty((splits, M, N), torch.float32, x.device, alloc)
    L = ops.lib("gemv_fused.cu")
    build.check(L, L.mlb_gemv_split(x.data_ptr(), x.stride(0), weight.data_ptr(), weight.stride(0), N, ops._ptr(bias),
                                    partial.data_ptr(), M, N, K, splits, k_per_cta, ops._stream()))
    return partial


def gemv_silu_mul(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, I] (bf16) = silu(x @ weight[:I]^T) * (x @ weight[I:2I]^T), one kernel, no partial sums."""
    M, K = x.shape
    I = out.shape[1]
    if weight.shape != (2 * I, K) or out.shape[0] != M or out.dtype != torch.bfloat16 or out.stride(1) != 1:
        raise KernelError("gemv_silu_mul: the weight must hold gate rows then up rows, the output be bf16 [M, I]")
    L = ops.lib("gemv_fused.cu")
    build.check(L, L.mlb_gemv_silu(x.data_ptr(), x.stride(0), weight.data_ptr(), weight.stride(0), 2 * I, I, out.data_ptr(),
                                   out.stride(0), M, I, K, ops._stream()))


def gemv_qkv_rope(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], positions: torch.Tensor,
                  token_seq: torch.Tensor, block_table: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor],
                  q_out: torch.Tensor, pages: Optional[torch.Tensor], num_heads: int, num_kv_heads: int, head_dim: int,
                  error_flag: Optional[torch.Tensor]) -> None:
    """Fused q/k/v projection of a few tokens with bias, split-half rotation over the whole head
    (inv_freq None: no rotation) and the store of keys and values into the paged cache
    (`pages` None: they are dropped); rotated queries go to q_out [M, NH*D] bf16."""
    M, K = x.shape
    width = (num_heads + 2 * num_kv_heads) * head_dim
    if weight.shape != (width, K) or q_out.shape != (M, num_heads * head_dim) or q_out.dtype != torch.bfloat16 \
            or not q_out.is_contiguous() or positions.shape[0] != M:
        raise KernelError("gemv_qkv_rope: shapes do not agree")
    if head_dim % 16:
        raise KernelError(f"gemv_qkv_rope: head_dim {head_dim} must be a multiple of 16")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.shape[0] * 2 != head_dim):
        raise KernelError("gemv_qkv_rope: inv_freq must hold head_dim/2 fp32 entries")
    if bias is not None and (bias.dtype != torch.float32 or bias.shape[0] != width):
        raise KernelError("gemv_qkv_rope: the bias must be fp32 of the fused width")
    num_pages = page_size = max_blocks = 0
    if pages is not None:
        num_pages, two, nkv, page_size, d = pages.shape
        if two != 2 or nkv != num_kv_heads or d != head_dim or pages.dtype != torch.bfloat16 or not pages.is_contiguous():
            raise KernelError(f"gemv_qkv_rope: pages {tuple(pages.shape)} do not match the head geometry")
        max_blocks = block_table.shape[1]
    L = ops.lib("gemv_fused.cu")
    build.check(L, L.mlb_gemv_qkv_rope(
        x.data_ptr(), x.stride(0), weight.data_ptr(), weight.stride(0), ops._ptr(bias), positions.data_ptr(),
        token_seq.data_ptr(), ops._ptr(block_table), max_blocks, ops._ptr(inv_freq), 1 if inv_freq is not None else 0,
        q_out.data_ptr(), ops._ptr(pages), num_pages, page_size, M, K, num_heads, num_kv_heads, head_dim,
        ops._ptr(error_flag), ops._stream()))


# ------------------------------------------------------------------------------ 9 to 128 tokens: tcgen05 weight streaming
STREAM_MAX_TOKENS = 128               # the token side of one tcgen05.mma tile
STREAM_MIN_K_BLOCKS_PER_SPLIT = 4     # 256 elements of K per CTA at least
STREAM_MAX_SPLITS = 16


def stream_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """What TMA can address: K and the row pitches multiples of 8 elements, bases 16-byte aligned."""
    m, k = x.shape
    return (0 < m <= STREAM_MAX_TOKENS and k % 8 == 0 and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0
            and x.stride(1) == 1 and weight.stride(1) == 1 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0
            and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16)


STREAM_SMALL_PRODUCT_BYTES = 8 << 20  # a weight of fewer bytes is a "small" product (QKV, O of a small model)
STREAM_SMALL_PRODUCT_MAX_TOKENS = 32  # measured at 64 tokens: the library's small products take 4.1 us, this kernel's 6.0


def stream_preferred(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """The tcgen05 streaming kernel can take this product and is the faster way for it: any product up to 32
    tokens; beyond that only the large ones, whose time is the weight stream (a small product is a few dependent
    round trips long, and there the partial results of its K split cost more than the library's way)."""
    m = x.shape[0]
    if not (m <= STREAM_MAX_TOKENS and stream_supported(x, weight)):
        return False
    if m <= GEMV_ROUTE_MAX_TOKENS:
        return not gemv_preferred(x, weight)
    return m <= STREAM_SMALL_PRODUCT_MAX_TOKENS or weight.numel() * weight.element_size() >= STREAM_SMALL_PRODUCT_BYTES


def stream_splits(n: int, k: int, sms: int = DEFAULT_SM_COUNT) -> int:
    """K ranges per 128-row tile: as many as give every SM a CTA, each at least 256 elements of K long, none empty."""
    tiles = -(-n // 128)
    k_blocks = -(-k // 64)
    splits = max(1, min(sms // tiles, k_blocks // STREAM_MIN_K_BLOCKS_PER_SPLIT, STREAM_MAX_SPLITS))
    per = -(-k_blocks // splits)
    return -(-k_blocks // per)


def stream_partials(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, splits: Optional[int] = None,
                    stages: int = 0, error_flag: Optional[torch.Tensor] = None, alloc=None) -> torch.Tensor:
    """[S, M, N] fp32 partial results of x @ weight^T (+ bias, in partial 0) from the tcgen05 streaming kernel."""
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K:
        raise KernelError(f"stream_partials: shapes {tuple(x.shape)} x {tuple(weight.shape)}^T do not agree")
    if bias is not None and (bias.dtype != torch.float32 or bias.shape[0] != N):
        raise KernelError("stream_partials: the bias must be fp32 of length N")
    L = ops.lib("gemm_stream.cu")
    splits = L.mlb_gemm_stream_splits(K, splits if splits is not None else stream_splits(N, K, sm_count(x.device)))
    shape = (splits, M, N)
    partial = alloc(shape, torch.float32) if alloc is not None else torch.empty(shape, dtype=torch.float32, device=x.device)
    flag = error_flag if error_flag is not None else device_error_flag(x.device)
    build.check(L, L.mlb_gemm_stream(x.data_ptr(), x.stride(0), weight.data_ptr(), weight.stride(0), N, ops._ptr(bias),
                                     partial.data_ptr(), M, N, K, splits, int(stages), flag.data_ptr(), ops._stream()))
    return partial


def stream_silu_mul(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, stages: int = 0,
                    error_flag: Optional[torch.Tensor] = None) -> None:
    """out[M, I] (bf16) = silu(x @ weight[:I]^T) * (x @ weight[I:2I]^T), the activation as the product's epilogue."""
    M, K = x.shape
    I = out.shape[1]
    if weight.shape != (2 * I, K) or out.shape[0] != M or out.dtype != torch.bfloat16 or out.stride(1) != 1:
        raise KernelError("stream_silu_mul: the weight must hold gate rows then up rows, the output be bf16 [M, I]")
    flag = error_flag if error_flag is not None else device_error_flag(x.device)
    L = ops.lib("gemm_stream.cu")
    build.check(L, L.mlb_gemm_stream_silu(x.data_ptr(), x.stride(0), weight.data_ptr(), weight.stride(0), 2 * I, I,
                                          out.data_ptr(), out.stride(0), M, I, K, int(stages), flag.data_ptr(), ops._stream()))


# ------------------------------------------------------------------------------ prompt portions: CTA pairs
def device_error_flag(device) -> torch.Tensor:
    """Where the tensor-memory kernels raise a code when one of their bounded waits ran out and the caller named
    no flag of its own (a part run outside a step).  Inside a step the parts pass the step's flag."""
    key = str(device)
    if key not in _error_flags:
        _error_flags[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_flags[key]


error_flag = device_error_flag


def supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    k = x.shape[1]
    return (k % 8 == 0 and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0
            and x.stride(1) == 1 and weight.stride(1) == 1 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def gemm_pair(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
              accumulate: bool = False, dual_rows: Optional[int] = None, stages: int = 0, sms: Optional[int] = None,
              error_flag: Optional[torch.Tensor] = None) -> None:
    """The CTA-pair tcgen05 product (`gemm_tc2.cu`) for prompt-sized token counts:
    out[M, N] = x[M, K] @ weight[:N]^T (+ bias) (+ out), or with dual_rows = I:
    out[M, I] = silu(x @ weight[:I]^T) * (x @ weight[I:2I]^T)."""
    M, K = x.shape
    dual = dual_rows is not None
    N = dual_rows if dual else weight.shape[0]
    if weight.shape[1] != K or out.shape != (M, N) or out.stride(1) != 1:
        raise KernelError(f"gemm_pair: shapes {tuple(x.shape)} x {tuple(weight.shape)}^T -> {tuple(out.shape)} do not agree")
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or out.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError("gemm_pair: bf16 operands and an fp32 or bf16 output are expected")
    if dual and weight.shape[0] < 2 * N:
        raise KernelError("gemm_pair: a dual product needs gate rows followed by up rows")
    flag = error_flag if error_flag is not None else device_error_flag(x.device)
    sms = sms if sms is not None else sm_count(x.device)
    sms -= sms % 2                                      # whole pairs
    L = ops.lib("gemm_tc2.cu")
    build.check(L, L.mlb_gemm_pair(x.data_ptr(), x.stride(0), weight.data_ptr(), weight.stride(0), weight.shape[0],
                                   ops._ptr(bias), out.data_ptr(), out.stride(0), 1 if out.dtype == torch.bfloat16 else 0,
                                   1 if accumulate else 0, 1 if dual else 0, N if dual else 0, M, N, K, int(stages),
                                   int(sms), flag.data_ptr(), ops._stream()))


def _direct_library(device) -> bool:
    """Whether cuBLASLt can be called without the tensor framework in between (csrc/gemm_lib.cu)."""
    global _direct_ok
    if _direct_ok is None:
        _direct_ok = bool(ops.lib("gemm_lib.cu").mlb_lt_available())
    return _direct_ok


def library_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype,
                   out: Optional[torch.Tensor], alloc=None) -> torch.Tensor:
    """cuBLASLt: bf16 operands, fp32 accumulate, output written in out_dtype.  `alloc(shape, dtype)` supplies
    the output when `out` is not given (default: a new tensor)."""
    LaunchCounter.library += 1
    if (bias is None and x.is_cuda and x.stride(1) == 1 and weight.stride(1) == 1 and x.shape[0] > 0
            and (out is None or (out.dtype == out_dtype and out.stride(1) == 1)) and _direct_library(x.device)):
        M, K = x.shape
        N = weight.shape[0]
        if out is None:
            out = alloc((M, N), out_dtype) if alloc is not None else torch.empty((M, N), dtype=out_dtype, device=x.device)
        key = str(x.device)
        work = _workspaces.get(key)
        if work is None:
            work = _workspaces[key] = torch.empty(LIBRARY_WORKSPACE_BYTES, dtype=torch.uint8, device=x.device)
        L = ops.lib("gemm_lib.cu")
        build.check(L, L.mlb_lt_matmul(x.data_ptr(), x.stride(0), weight.data_ptr(), weight.stride(0), out.data_ptr(),
                                       out.stride(0), 1 if out_dtype == torch.bfloat16 else 0, 0, M, N, K,
                                       work.data_ptr(), LIBRARY_WORKSPACE_BYTES, ops._stream()))
        return out
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


PAIR_MIN_TOKENS = 256                       # from here on the fused gate/up + activation of gemm_tc2 beats library + activation kernel


def linear_bf16(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype,
                out: Optional[torch.Tensor], partials_ok: bool = False, alloc=None,
                error_flag: Optional[torch.Tensor] = None) -> torch.Tensor:
    if partials_ok and out is None and out_dtype == torch.float32:
        if gemv_preferred(x, weight):
            return gemv_partials(x, weight, bias, alloc=alloc)
        if stream_preferred(x, weight):
            return stream_partials(x, weight, bias, error_flag=error_flag, alloc=alloc)
    return library_linear(x, weight, bias, out_dtype, out, alloc)
