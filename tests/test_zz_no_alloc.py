"""The few-token product that brings its own scratch memory (csrc/gemv_noalloc.h), called
through its exported C symbol the way a program that cannot allocate device memory would
call it, and compared with the regular entry point, which is handed scratch by its caller.

Collected last on purpose: a run that stops at the first failure has then already run every
other test."""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def library():
    from microllm_rocm_b200.kernels import build
    lib = build.load("gemv_noalloc.cu")
    lib.mlb_gemv_bf16_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_longlong,
                                          ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int,
                                          ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.mlb_gemv_bf16_noalloc.restype = ctypes.c_int
    lib.mlb_gemv_bf16_noalloc_scratch_needed.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int]
    lib.mlb_gemv_bf16_noalloc_scratch_needed.restype = ctypes.c_longlong
    return lib


def regular(x, w, bias):
    """The existing entry point: partial results in caller-provided scratch, added in split order."""
    from microllm_rocm_b200.kernels import gemm_bf16
    part = gemm_bf16.gemv_partials(x, w, bias)
    acc = part[0].clone()
    for s in range(1, part.shape[0]):
        acc += part[s]
    return acc


def call(lib, x, w, bias, out):
    stream = torch.cuda.current_stream().cuda_stream
    return lib.mlb_gemv_bf16_noalloc(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0),
                                     None if bias is None else bias.data_ptr(), out.data_ptr(), out.stride(0),
                                     x.shape[0], w.shape[0], x.shape[1], stream)


def test_no_alloc_product_matches_the_regular_one_on_two_calls_in_a_row():
    lib = library()
    torch.manual_seed(0)
    # the second call is smaller and uses fewer splits: anything the first left in the shared
    # scratch array would show up in it
    for M, N, K, with_bias in [(8, 1536, 8960, True), (3, 200, 96, False)]:
        x = torch.randn(M, K, device=DEV).bfloat16()
        w = torch.randn(N, K, device=DEV).bfloat16()
        bias = torch.randn(N, device=DEV) if with_bias else None
        out = torch.full((M, N), float("nan"), device=DEV)
        before = torch.cuda.memory_allocated()
        status = call(lib, x, w, bias, out)
        assert status == 0, lib.mlb_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before, "the call must not allocate through torch either"
        want = regular(x, w, bias)
        assert torch.isfinite(out).all()
        assert (out - want).abs().max().item() <= 2e-5 * math.sqrt(K) * 4
        exact = x.double() @ w.double().t() + (bias.double() if with_bias else 0)
        assert (out.double() - exact).abs().max().item() <= 2e-5 * math.sqrt(K) * 4


def test_no_alloc_product_refuses_what_its_scratch_cannot_hold():
    lib = library()
    limit = 4 << 20
    assert lib.mlb_gemv_bf16_noalloc_scratch_needed(8, 1536, 8960) <= limit
    assert lib.mlb_gemv_bf16_noalloc_scratch_needed(16, 400000, 64) > limit
    x = torch.zeros(16, 64, device=DEV).bfloat16()
    w = torch.zeros(8, 64, device=DEV).bfloat16()          # never read: the size check comes first
    out = torch.zeros(16, 8, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    status = lib.mlb_gemv_bf16_noalloc(x.data_ptr(), 64, w.data_ptr(), 64, None, out.data_ptr(), 400000, 16, 400000, 64, stream)
    assert status != 0
    message = lib.mlb_last_error().decode()
    assert "scratch" in message and "mlb_gemv_bf16" in message
    assert lib.mlb_gemv_bf16_noalloc(x.data_ptr(), 64, w.data_ptr(), 64, None, out.data_ptr(), 8, 17, 8, 64, stream) != 0
    assert "1..16" in lib.mlb_last_error().decode()
    # a missing operand is an error code on the host, never an address for the kernel
    for args in [(None, w.data_ptr(), out.data_ptr()), (x.data_ptr(), None, out.data_ptr()), (x.data_ptr(), w.data_ptr(), None)]:
        assert lib.mlb_gemv_bf16_noalloc(args[0], 64, args[1], 64, None, args[2], 8, 16, 8, 64, stream) == 1
        assert "null" in lib.mlb_last_error().decode()
    torch.cuda.synchronize()
