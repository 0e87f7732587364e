"""Matrix products of the projections: y[M,N] = x[M,K] @ W[N,K]^T (+ bias).

fp32 path: the hand-written CUDA-core kernel (`gemm_f32.cu`), plain fp32 FMA, fixed
summation order.  bf16 path: bf16 operands with fp32 accumulation; the library product
(cuBLASLt, see gemm_bf16.library_linear) stands where the reference calls hipBLASLt for the same
projections (src/ops/optimized.cpp:349-403, BF16 x BF16 with 32-bit compute), and the
hand-written weight-streaming kernels take over for steps of up to 128 tokens.
Weights stay in the checkpoint's [out, in] layout.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops
from .build import KernelError


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: torch.dtype = torch.float32, out: Optional[torch.Tensor] = None,
           partials_ok: bool = False, alloc=None, error_flag: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [M,K] and weight [N,K] in the same dtype (f32 or bf16); returns [M,N] in `out_dtype`.
    With partials_ok the caller accepts [S, M, N] fp32 partial results instead (a product whose
    K range was split over CTAs) and adds them up itself, in order, where it reads them.
    `alloc(shape, dtype)`: where a plain [M,N] result comes from when `out` is not given (a step's scratch).
    `error_flag`: the step's device flag, raised by a tensor-memory kernel whose bounded wait ran out."""
    if x.dtype != weight.dtype:
        raise KernelError(f"linear: activations are {x.dtype} but the weight is {weight.dtype}")
    M, N = x.shape[0], weight.shape[0]
    if x.dtype == torch.float32:
        if out_dtype != torch.float32:
            raise KernelError("linear: the fp32 path produces fp32")
        if out is None:
            out = alloc((M, N), torch.float32) if alloc is not None else torch.empty((M, N), dtype=torch.float32, device=x.device)
        ops.gemm_f32(x, weight, out, bias=bias)
        return out
    if x.dtype != torch.bfloat16:
        raise KernelError(f"linear: unsupported dtype {x.dtype}")
    if not x.is_cuda:
        raise KernelError("linear: there is no CPU path")
    from . import gemm_bf16
    return gemm_bf16.linear_bf16(x, weight, bias, out_dtype, out, partials_ok=partials_ok, alloc=alloc, error_flag=error_flag)
