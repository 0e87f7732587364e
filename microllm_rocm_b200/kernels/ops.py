"""Python faces of the CUDA kernels: each function checks what it is given, then launches
on torch's current stream through the library's C ABI.  Tensors are torch CUDA tensors
used as typed device memory; no torch operator computes anything here.

There is no CPU path and no silent fallback: a missing compiler or extension raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import build
from .build import KernelError

F32, BF16 = 0, 1
_DTYPE_TAG = {torch.float32: F32, torch.bfloat16: BF16}


def dtype_tag(t: torch.Tensor) -> int:
    try:
        return _DTYPE_TAG[t.dtype]
    except KeyError:
        raise KernelError(f"unsupported tensor dtype {t.dtype}") from None


# The current stream's handle straight from the runtime's binding: the Stream object that
# torch.cuda.current_stream() builds costs more host time than a short kernel runs.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_current_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    if _raw_stream is not None and _current_device is not None:
        return _raw_stream(_current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, name: str, dtype=None, dims: Optional[int] = None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name} must have {dims} dimensions, got {tuple(t.shape)}")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


_SIGNATURES = {
    "basic.cu": {
        "mlb_embed_gather": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "mlb_rmsnorm": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p],
        "mlb_add_rmsnorm": [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
        "mlb_scatter_int": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p],
        "mlb_stream_fork": [c_void_p, c_void_p],
        "mlb_stream_join": [c_void_p, c_void_p],
        "mlb_add_inplace": [c_void_p, c_void_p, c_int, c_longlong, c_longlong, c_void_p],
        "mlb_silu_mul": [c_void_p, c_void_p, c_longlong, c_int, c_int, c_longlong, c_void_p, c_int, c_int, c_int, c_void_p],
        "mlb_cast_f32_bf16": [c_void_p, c_void_p, c_longlong, c_void_p],
        "mlb_copy_async": [c_void_p, c_void_p, c_longlong, c_int, c_void_p],
        "mlb_stream_synchronize": [c_void_p],
        "mlb_decode_advance": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    },
    "gemm_f32.cu": {
        "mlb_gemm_f32": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                         c_longlong, c_longlong, c_longlong, c_int, c_void_p],
    },
    "rope_kv.cu": {
        "mlb_rope_kv_write": [c_void_p, c_longlong, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                              c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                              c_int, c_int, c_int, c_void_p, c_void_p, c_void_p],
        "mlb_rope_table": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    },
    "attention_plain.cu": {
        "mlb_paged_attention_plain": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                      c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                      c_float, c_void_p, c_void_p],
    },
    "sampling.cu": {
        "mlb_argmax_rows": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p],
        "mlb_sample_rows": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                            c_void_p, c_void_p],
    },
}

_libs = {}


# Further -D definitions per source, merged into what a caller asks for.  Empty in the product; tests load the
# warp-specialised kernels with one warp held back (MLB_LAG_WARP, csrc/common.cuh) through it.
TEST_DEFINES: dict = {}


def lagged_sources():
    """The held-back builds the tests ask for, so that the build check compiles them too and no test waits for nvcc:
    every role of every kernel whose warps meet at mbarriers (copy, MMA issue, one epilogue or softmax warp)."""
    out = [("attention_tc.cu", {"HEAD_DIM": 128, "MLB_LAG_WARP": w}) for w in (0, 1, 2, 5)]
    out += [("gemm_stream.cu", {"MLB_LAG_WARP": w}) for w in (0, 1, 3)]
    out += [("gemm_tc2.cu", {"MLB_LAG_WARP": w, "MLB_LAG_RANK": r}) for w, r in ((0, 1), (1, 0), (3, 0), (4, 1))]
    out += [("attention_mma.cu", {"HEAD_DIM": 128, "MLB_LAG_WARP": w}) for w in (1, 4)]
    return out


def lib(source: str, defines=None) -> ctypes.CDLL:
    if TEST_DEFINES.get(source):
        defines = {**(defines or {}), **TEST_DEFINES[source]}
    key = (source, tuple(sorted((defines or {}).items())))
    got = _libs.get(key)
    if got is None:
        got = build.load(source, defines)
        from .replay import Launcher
        for name, argtypes in _SIGNATURES.get(source, {}).items():
            fn = getattr(got, name)
            if isinstance(fn, Launcher):
                continue
            fn.argtypes = argtypes
            fn.restype = c_int
            if argtypes and argtypes[-1] is c_void_p:
                # a launcher (its last argument is the stream): calls through; a recorder may listen (kernels/replay.py).
                # Queries (split counts, limits) return numbers, not a status, and are never recorded.
                setattr(got, name, Launcher(got, fn, argtypes))
        _libs[key] = got
    return got


def register_signatures(source: str, signatures) -> None:
    _SIGNATURES.setdefault(source, {}).update(signatures)


def base_sources():
    """(source, defines) of every kernel that any model needs."""
    return [("basic.cu", {}), ("gemm_f32.cu", {}), ("rope_kv.cu", {}), ("attention_plain.cu", {}),
            ("sampling.cu", {}), ("replay.cu", {})]


def all_sources():
    """Every object the package can ask for with its default head sizes: what the build
    check compiles."""
    from . import attention
    out = base_sources()
    for d in (32, 64, 128):
        out += attention.mma_sources(d) + attention.tc_sources(d)
    from . import gemm_bf16
    return out + gemm_bf16.sources() + [("gemv_noalloc.cu", {})]


# ------------------------------------------------------------------------------ basic
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> None:
    _need(table, "table", dims=2); _need(ids, "ids", torch.int32, 1); _need(out, "out", torch.float32, 2)
    vocab, width = table.shape
    if out.shape != (ids.shape[0], width):
        raise KernelError(f"embed_gather: out {tuple(out.shape)} does not match ({ids.shape[0]}, {width})")
    L = lib("basic.cu")
    build.check(L, L.mlb_embed_gather(table.data_ptr(), dtype_tag(table), ids.data_ptr(), out.data_ptr(),
                                      ids.shape[0], width, vocab, _stream()))


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = rmsnorm(x[rows[r]] if rows is given else x[r])."""
    _need(x, "x", torch.float32, 2); _need(weight, "weight", torch.float32, 1); _need(out, "out", dims=2)
    width = x.shape[1]
    n = rows.shape[0] if rows is not None else x.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
    if weight.shape[0] != width or out.shape != (n, width):
        raise KernelError("rmsnorm: shapes do not agree")
    L = lib("basic.cu")
    build.check(L, L.mlb_rmsnorm(x.data_ptr(), weight.data_ptr(), out.data_ptr(), dtype_tag(out), _ptr(rows),
                                 n, width, float(eps), _stream()))


def _partials(delta: torch.Tensor, shape, name: str):
    """A delta is [M, N] or, from a product split over K, [S, M, N]: (count, stride in elements)."""
    _need(delta, name, torch.float32)
    if delta.dim() == 3 and tuple(delta.shape[1:]) == tuple(shape):
        return delta.shape[0], delta.shape[1] * delta.shape[2]
    if tuple(delta.shape) == tuple(shape):
        return 1, 0
    raise KernelError(f"{name}: shape {tuple(delta.shape)} is neither {tuple(shape)} nor [splits, {', '.join(map(str, shape))}]")


def add_rmsnorm(residual: torch.Tensor, delta: torch.Tensor, weight: torch.Tensor, eps: float,
                out: torch.Tensor) -> None:
    """residual += delta (in place, fp32; a [S, M, N] delta is summed over S in order), then
    out = rmsnorm(residual)."""
    _need(residual, "residual", torch.float32, 2)
    _need(weight, "weight", torch.float32, 1); _need(out, "out", dims=2)
    n_delta, stride = _partials(delta, residual.shape, "add_rmsnorm delta")
    if out.shape != residual.shape or weight.shape[0] != residual.shape[1]:
        raise KernelError("add_rmsnorm: shapes do not agree")
    L = lib("basic.cu")
    build.check(L, L.mlb_add_rmsnorm(residual.data_ptr(), delta.data_ptr(), n_delta, stride, weight.data_ptr(),
                                     out.data_ptr(), dtype_tag(out), residual.shape[0], residual.shape[1], float(eps),
                                     _stream()))


def add_inplace(x: torch.Tensor, delta: torch.Tensor) -> None:
    """x += delta; a [S, ...] stack of partial results is summed over S in order."""
    _need(x, "x", torch.float32)
    n_delta, stride = _partials(delta, x.shape, "add_inplace delta")
    L = lib("basic.cu")
    build.check(L, L.mlb_add_inplace(x.data_ptr(), delta.data_ptr(), n_delta, stride, x.numel(), _stream()))


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[r, c] = silu(gate_up[r, c]) * gate_up[r, width + c] for a fused [rows, 2*width] input, or
    for its [S, rows, 2*width] partial results (summed over S in order first)."""
    _need(out, "out", dims=2)
    rows, width = out.shape
    n_partials, partial_stride = 1, 0
    if gate_up.dim() == 3:
        _need(gate_up, "gate_up", dims=3)
        n_partials, partial_stride = gate_up.shape[0], gate_up.shape[1] * gate_up.shape[2]
        first = gate_up[0]
    else:
        _need(gate_up, "gate_up", dims=2)
        first = gate_up
    if first.shape != (rows, 2 * width):
        raise KernelError("silu_mul: input must be [rows, 2*width]")
    L = lib("basic.cu")
    esz = gate_up.element_size()
    build.check(L, L.mlb_silu_mul(gate_up.data_ptr(), gate_up.data_ptr() + width * esz, 2 * width,
                                  dtype_tag(gate_up), n_partials, partial_stride, out.data_ptr(), dtype_tag(out), rows,
                                  width, _stream()))


def cast_f32_bf16(x: torch.Tensor, out: torch.Tensor) -> None:
    _need(x, "x", torch.float32); _need(out, "out", torch.bfloat16)
    if x.numel() != out.numel():
        raise KernelError("cast: sizes differ")
    L = lib("basic.cu")
    build.check(L, L.mlb_cast_f32_bf16(x.data_ptr(), out.data_ptr(), x.numel(), _stream()))


def decode_advance(positions: torch.Tensor, seq_pos0: torch.Tensor, seq_lens: torch.Tensor, draw: torch.Tensor,
                   tokens: Optional[torch.Tensor] = None, error_flag: Optional[torch.Tensor] = None,
                   result: Optional[torch.Tensor] = None, grows: Optional[torch.Tensor] = None) -> None:
    """Every sequence of a captured decode step has grown by one token: advance its position,
    extents and draw counter on the device.  With `result` ([n + 1] int32) the step's selected
    `tokens` and the error flag are gathered there, for one device -> host copy.  `grows` ([n] int32 of
    1 and 0): rows with 0 stay where they are (rows that only fill a captured batch up)."""
    n = positions.shape[0]
    _need(positions, "positions", torch.int32, 1); _need(seq_pos0, "seq_pos0", torch.int32, 1)
    _need(seq_lens, "seq_lens", torch.int32, 1); _need(draw, "draw", torch.int64, 1)
    if not (seq_pos0.shape[0] == seq_lens.shape[0] == draw.shape[0] == n):
        raise KernelError("decode_advance: one entry per sequence in every array")
    if result is not None:
        _need(result, "result", torch.int32, 1); _need(tokens, "tokens", torch.int32, 1)
        if result.shape[0] != n + 1 or tokens.shape[0] != n:
            raise KernelError("decode_advance: result holds one int per sequence and one more for the error flag")
    if grows is not None:
        _need(grows, "grows", torch.int32, 1)
        if grows.shape[0] != n:
            raise KernelError("decode_advance: one growth per sequence")
    L = lib("basic.cu")
    build.check(L, L.mlb_decode_advance(positions.data_ptr(), seq_pos0.data_ptr(), seq_lens.data_ptr(), draw.data_ptr(),
                                        n, _ptr(tokens), _ptr(error_flag), _ptr(result), _ptr(grows), _stream()))


def copy_async(dst: torch.Tensor, src: torch.Tensor) -> None:
    """A small contiguous copy between pinned host memory and the device on the current stream, through the
    runtime directly (a tensor library's copy costs several microseconds of dispatch for a few bytes)."""
    nbytes = src.numel() * src.element_size()
    if dst.numel() * dst.element_size() != nbytes or not dst.is_contiguous() or not src.is_contiguous():
        raise KernelError("copy_async: both sides must be contiguous and of the same size")
    if dst.is_cuda == src.is_cuda:
        raise KernelError("copy_async: one side on the device, the other in pinned host memory")
    host = src if dst.is_cuda else dst
    if not host.is_pinned():
        raise KernelError("copy_async: the host side must be pinned")
    L = lib("basic.cu")
    status = L.mlb_copy_async(dst.data_ptr(), src.data_ptr(), nbytes, 1 if dst.is_cuda else 0, _stream())
    if status != 0:
        build.check(L, status)


def copy_raw(dst: int, src: int, nbytes: int, to_device: bool) -> None:
    """`copy_async` for a caller that keeps the two addresses of buffers it owns (pinned host, device)."""
    L = lib("basic.cu")
    status = L.mlb_copy_async(dst, src, nbytes, 1 if to_device else 0, _stream())
    if status != 0:
        build.check(L, status)


# ------------------------------------------------------------------------------ small host -> device uploads
# A copy from pageable host memory makes the runtime wait for everything queued on the stream before it stages the
# data: a step that is issued while the step before it still runs would stall at its first small upload (a work
# list, a row of sampling parameters).  These go through a ring of pinned slots instead and never wait for the GPU.
_UPLOAD_SLOTS, _UPLOAD_SLOT_BYTES = 32, 64 << 10
_staging = {}
_NUMPY_TO_TORCH = {"int32": torch.int32, "int64": torch.int64, "float32": torch.float32}


def upload(values, dtype: str, device: torch.device) -> torch.Tensor:
    """A new device tensor holding `values` (a sequence or array; dtype 'int32', 'int64' or 'float32'), copied
    asynchronously out of pinned memory on the current stream."""
    import numpy as np
    array = np.ascontiguousarray(np.asarray(values, dtype=dtype))
    out = torch.empty(array.shape, dtype=_NUMPY_TO_TORCH[dtype], device=device)
    if array.size == 0:
        return out
    if array.nbytes > _UPLOAD_SLOT_BYTES:
        out.copy_(torch.from_numpy(array).pin_memory(), non_blocking=True)       # rare: too large for a slot
        return out
    key = str(device)
    ring = _staging.get(key)
    if ring is None:
        ring = _staging[key] = {"pinned": torch.empty((_UPLOAD_SLOTS, _UPLOAD_SLOT_BYTES), dtype=torch.uint8, pin_memory=True),
                                "events": [None] * _UPLOAD_SLOTS, "next": 0}
    i = ring["next"]
    ring["next"] = (i + 1) % _UPLOAD_SLOTS
    if ring["events"][i] is not None:
        ring["events"][i].synchronize()              # the copy that last read this slot (many uploads ago) has run
    host = ring["pinned"][i, :array.nbytes].view(_NUMPY_TO_TORCH[dtype]).reshape(array.shape)
    host.numpy()[...] = array
    out.copy_(host, non_blocking=True)
    event = ring["events"][i] or torch.cuda.Event()
    event.record()
    ring["events"][i] = event
    return out


def scatter_int(dst: torch.Tensor, dst_index: torch.Tensor, src: torch.Tensor, src_index: torch.Tensor) -> None:
    """dst[dst_index[i]] = src[src_index[i]] for int32 arrays on the device (indices outside an array are skipped)."""
    for name, t in (("dst", dst), ("dst_index", dst_index), ("src", src), ("src_index", src_index)):
        _need(t, name, torch.int32, 1)
    if dst_index.shape[0] != src_index.shape[0]:
        raise KernelError("scatter_int: one source index per destination index")
    L = lib("basic.cu")
    build.check(L, L.mlb_scatter_int(dst.data_ptr(), dst.shape[0], dst_index.data_ptr(), src.data_ptr(), src.shape[0],
                                     src_index.data_ptr(), dst_index.shape[0], _stream()))


_side_streams = {}


def side_stream() -> int:
    """This device's second stream, for work of a step that is independent of what the main stream does meanwhile
    (see fork / join)."""
    device = _current_device() if _current_device is not None else torch.cuda.current_device()
    handle = _side_streams.get(device)
    if handle is None:
        L = lib("basic.cu")
        L.mlb_side_stream.restype = c_void_p
        L.mlb_side_stream.argtypes = []
        handle = L.mlb_side_stream()
        if not handle:
            raise KernelError("the device's second stream could not be made")
        _side_streams[device] = handle
    return handle


def fork(side: int) -> None:
    """The side stream continues from where the current stream stands."""
    L = lib("basic.cu")
    build.check(L, L.mlb_stream_fork(side, _stream()))


def join(side: int) -> None:
    """The current stream waits for everything queued on the side stream."""
    L = lib("basic.cu")
    build.check(L, L.mlb_stream_join(side, _stream()))


def stream_synchronize() -> None:
    L = lib("basic.cu")
    status = L.mlb_stream_synchronize(_stream())
    if status != 0:
        build.check(L, status)


# ------------------------------------------------------------------------------ fp32 GEMM
def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
             accumulate: bool = False) -> None:
    """out[M,N] (+)= a[M,K] @ w[N,K]^T (+ bias[N]); plain fp32 FMA on CUDA cores."""
    _need(a, "a", torch.float32, 2); _need(w, "w", torch.float32, 2); _need(out, "out", torch.float32, 2)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm_f32: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} do not agree")
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
        if bias.shape[0] != N:
            raise KernelError("gemm_f32: bias length differs from N")
    L = lib("gemm_f32.cu")
    build.check(L, L.mlb_gemm_f32(a.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), M, N, K, K, K, N,
                                  1 if accumulate else 0, _stream()))


# ------------------------------------------------------------------------------ rope + kv store
def rope_kv_write(qkv: torch.Tensor, bias: Optional[torch.Tensor], positions: torch.Tensor,
                  token_seq: torch.Tensor, block_table: Optional[torch.Tensor], inv_freq: torch.Tensor,
                  rot_dim: int, interleaved: bool, q_out: torch.Tensor, pages: Optional[torch.Tensor],
                  num_heads: int, num_kv_heads: int, head_dim: int, error_flag: Optional[torch.Tensor],
                  cos_sin: Optional[torch.Tensor] = None) -> None:
    """Bias, rotation and the K/V store for a fused [T, (NH+2NKV)*D] fp32 projection output
    (or its [S, T, width] partial results, which are summed here).
    `pages` is [num_pages, 2, NKV, page_size, D]; None makes the call query-only.
    `cos_sin` [T, rot_dim/2, 2] fp32 (from `rope_table`) spares the kernel the sines and cosines."""
    _need(positions, "positions", torch.int32, 1)
    n_partials, partial_stride = 1, 0
    if qkv.dim() == 3:
        _need(qkv, "qkv", torch.float32, 3)
        n_partials, partial_stride = qkv.shape[0], qkv.shape[1] * qkv.shape[2]
        qkv = qkv[0]
    _need(qkv, "qkv", torch.float32, 2)
    _need(token_seq, "token_seq", torch.int32, 1); _need(inv_freq, "inv_freq", torch.float32, 1)
    _need(q_out, "q_out", dims=2)
    T = qkv.shape[0]
    width = (num_heads + 2 * num_kv_heads) * head_dim
    if qkv.shape[1] != width or q_out.shape != (T, num_heads * head_dim) or positions.shape[0] != T:
        raise KernelError("rope_kv_write: shapes do not agree")
    if inv_freq.shape[0] * 2 != rot_dim:
        raise KernelError("rope_kv_write: inv_freq must have rot_dim/2 entries")
    if cos_sin is not None and (cos_sin.dtype != torch.float32 or tuple(cos_sin.shape) != (T, rot_dim // 2, 2)
                                or not cos_sin.is_contiguous()):
        raise KernelError("rope_kv_write: cos_sin must be a contiguous fp32 [T, rot_dim/2, 2] table")
    num_pages = page_size = max_blocks = 0
    if pages is not None:
        _need(pages, "pages", dims=5); _need(block_table, "block_table", torch.int32, 2)
        num_pages, two, nkv, page_size, d = pages.shape
        if two != 2 or nkv != num_kv_heads or d != head_dim:
            raise KernelError(f"rope_kv_write: pages {tuple(pages.shape)} do not match the head geometry")
        max_blocks = block_table.shape[1]
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
        if bias.shape[0] != width:
            raise KernelError("rope_kv_write: bias length differs from the fused width")
    L = lib("rope_kv.cu")
    build.check(L, L.mlb_rope_kv_write(
        qkv.data_ptr(), width, n_partials, partial_stride, _ptr(bias), positions.data_ptr(), token_seq.data_ptr(), _ptr(block_table), max_blocks,
        inv_freq.data_ptr(), rot_dim, 1 if interleaved else 0, q_out.data_ptr(), dtype_tag(q_out),
        _ptr(pages), dtype_tag(pages) if pages is not None else F32, num_pages, page_size, T,
        num_heads, num_kv_heads, head_dim, _ptr(error_flag), _ptr(cos_sin), _stream()))


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """[T, len(inv_freq), 2] fp32: (cos, sin) of position * inverse frequency, the rotation kernels' own
    fp32 expressions; made once per step and shared by every layer."""
    _need(positions, "positions", torch.int32, 1); _need(inv_freq, "inv_freq", torch.float32, 1)
    shape = (positions.shape[0], inv_freq.shape[0], 2)
    if out is None:
        out = torch.empty(shape, dtype=torch.float32, device=positions.device)
    else:
        _need(out, "out", torch.float32, 3)
        if tuple(out.shape) != shape:
            raise KernelError("rope_table: the output must be [T, len(inv_freq), 2]")
    L = lib("rope_kv.cu")
    build.check(L, L.mlb_rope_table(positions.data_ptr(), inv_freq.data_ptr(), out.data_ptr(), positions.shape[0],
                                    inv_freq.shape[0], _stream()))
    return out


# ------------------------------------------------------------------------------ attention
def paged_attention_plain(q: torch.Tensor, pages: torch.Tensor, out: torch.Tensor, positions: torch.Tensor,
                          token_seq: torch.Tensor, block_table: torch.Tensor, num_heads: int, num_kv_heads: int,
                          head_dim: int, scale: float, window: Optional[int],
                          error_flag: Optional[torch.Tensor]) -> None:
    _need(q, "q", dims=2); _need(pages, "pages", dims=5); _need(out, "out", dims=2)
    _need(positions, "positions", torch.int32, 1); _need(token_seq, "token_seq", torch.int32, 1)
    _need(block_table, "block_table", torch.int32, 2)
    T = q.shape[0]
    num_pages, two, nkv, page_size, d = pages.shape
    if two != 2 or nkv != num_kv_heads or d != head_dim:
        raise KernelError(f"paged_attention: pages {tuple(pages.shape)} do not match the head geometry")
    if q.shape[1] != num_heads * head_dim or out.shape != q.shape or positions.shape[0] != T:
        raise KernelError("paged_attention: shapes do not agree")
    L = lib("attention_plain.cu")
    build.check(L, L.mlb_paged_attention_plain(
        q.data_ptr(), dtype_tag(q), pages.data_ptr(), dtype_tag(pages), out.data_ptr(), dtype_tag(out),
        positions.data_ptr(), token_seq.data_ptr(), block_table.data_ptr(), block_table.shape[1], num_pages,
        page_size, T, num_heads, num_kv_heads, head_dim, int(window or 0), float(scale), _ptr(error_flag),
        _stream()))


# ------------------------------------------------------------------------------ sampling
def argmax_rows(logits: torch.Tensor, out: torch.Tensor) -> None:
    _need(logits, "logits", torch.float32, 2); _need(out, "out", torch.int32, 1)
    if out.shape[0] != logits.shape[0]:
        raise KernelError("argmax_rows: out length differs from the number of rows")
    L = lib("sampling.cu")
    build.check(L, L.mlb_argmax_rows(logits.data_ptr(), logits.shape[1], logits.shape[0], logits.shape[1],
                                     out.data_ptr(), _stream()))


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, seed: torch.Tensor,
                draw: torch.Tensor, out: torch.Tensor) -> None:
    """Per row: greedy when temperature == 0 or top_k == 1, else the seeded draw.  `seed` and
    `draw` are int64 tensors read as unsigned 64-bit."""
    _need(logits, "logits", torch.float32, 2); _need(out, "out", torch.int32, 1)
    _need(temperature, "temperature", torch.float32, 1); _need(top_k, "top_k", torch.int32, 1)
    _need(seed, "seed", torch.int64, 1); _need(draw, "draw", torch.int64, 1)
    R = logits.shape[0]
    if not (out.shape[0] == temperature.shape[0] == top_k.shape[0] == seed.shape[0] == draw.shape[0] == R):
        raise KernelError("sample_rows: per-row arrays must have one entry per logits row")
    L = lib("sampling.cu")
    build.check(L, L.mlb_sample_rows(logits.data_ptr(), logits.shape[1], R, logits.shape[1], temperature.data_ptr(),
                                     top_k.data_ptr(), seed.data_ptr(), draw.data_ptr(), out.data_ptr(), _stream()))
