"""Each kernel alone against a plain fp32 reference of the same operation, at sizes other
than the engine's tests use: widths and vocabularies that are no power of two, head sizes
from 16 to 256, odd group sizes.  Where random inputs would hide a fault the inputs are made
so that it shows (one far key that must dominate, the exact edge of a window, keys that sit
in the last slot of a page)."""
import math
import random

import numpy as np
import pytest
import torch

from tests.plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu

DEV = "cuda"


def ops():
    from microllm_rocm_b200.kernels import ops as o
    return o


def tol(dtype):
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


# ------------------------------------------------------------------------------ rows
@pytest.mark.parametrize("width", [16, 100, 1536, 5000])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_and_fused_add(width, out_dtype):
    torch.manual_seed(width)
    x = torch.randn(37, width) * 3
    w = 1 + 0.1 * torch.randn(width)
    d = torch.randn(37, width)
    eps = 1e-5
    want = plain.rms_norm(x, w, eps)
    out = torch.empty(37, width, dtype=out_dtype, device=DEV)
    ops().rmsnorm(x.to(DEV), w.to(DEV), eps, out)
    assert torch.allclose(out.float().cpu(), want, **tol(out_dtype))
    # selected rows only
    rows = torch.tensor([5, 0, 36, 5], dtype=torch.int32)
    out2 = torch.empty(4, width, dtype=out_dtype, device=DEV)
    ops().rmsnorm(x.to(DEV), w.to(DEV), eps, out2, rows=rows.to(DEV))
    assert torch.allclose(out2.float().cpu(), want[rows.long()], **tol(out_dtype))
    # residual += delta, then norm
    res = x.to(DEV).clone()
    ops().add_rmsnorm(res, d.to(DEV), w.to(DEV), eps, out)
    assert torch.equal(res.cpu(), x + d)
    assert torch.allclose(out.float().cpu(), plain.rms_norm(x + d, w, eps), **tol(out_dtype))


def test_rmsnorm_row_result_does_not_depend_on_the_batch():
    torch.manual_seed(0)
    x = torch.randn(64, 777, device=DEV)
    w = torch.randn(777, device=DEV)
    a = torch.empty_like(x)
    ops().rmsnorm(x, w, 1e-6, a)
    b = torch.empty(1, 777, device=DEV)
    ops().rmsnorm(x[13:14].contiguous(), w, 1e-6, b)
    assert torch.equal(a[13], b[0])


@pytest.mark.parametrize("table_dtype", [torch.float32, torch.bfloat16])
def test_embedding_gather_and_bad_id(table_dtype):
    torch.manual_seed(1)
    table = torch.randn(301, 70).to(table_dtype)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32)
    out = torch.empty(5, 70, device=DEV)
    ops().embed_gather(table.to(DEV), ids.to(DEV), out)
    assert torch.equal(out.cpu(), plain.embedding(table.float(), ids.tolist()))
    bad = torch.tensor([3, 301, -1], dtype=torch.int32, device=DEV)
    out = torch.empty(3, 70, device=DEV)
    ops().embed_gather(table.to(DEV), bad, out)
    assert torch.isfinite(out[0]).all() and torch.isnan(out[1]).all() and torch.isnan(out[2]).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_mul(dtype):
    torch.manual_seed(2)
    gu = (torch.randn(9, 2 * 173) * 4).to(dtype)
    gu[0, 0], gu[0, 1] = 90.0, -90.0                    # both branches of the stable sigmoid
    out = torch.empty(9, 173, dtype=dtype, device=DEV)
    ops().silu_mul(gu.to(DEV), out)
    want = plain.swiglu(gu[:, :173].float(), gu[:, 173:].float())
    assert torch.allclose(out.float().cpu(), want, **tol(dtype))


# ------------------------------------------------------------------------------ fp32 product
@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (3, 70, 33), (65, 129, 200), (130, 64, 17), (7, 1000, 1536)])
def test_gemm_f32_is_a_true_fp32_product(M, N, K):
    torch.manual_seed(M * N + K)
    a, w, bias = torch.randn(M, K), torch.randn(N, K), torch.randn(N)
    want = (a.double() @ w.double().t() + bias.double())
    out = torch.empty(M, N, device=DEV)
    ops().gemm_f32(a.to(DEV), w.to(DEV), out, bias=bias.to(DEV))
    err = (out.cpu().double() - want).abs().max()
    # fp32 accumulation over K terms: far below what a reduced-precision matrix mode gives
    assert err <= 2e-6 * math.sqrt(K) * 4, err
    base = torch.randn(M, N)
    acc = base.to(DEV).clone()
    ops().gemm_f32(a.to(DEV), w.to(DEV), acc, accumulate=True)
    assert torch.allclose(acc.cpu().double(), base.double() + a.double() @ w.double().t(), atol=2e-5 * math.sqrt(K))


def test_gemm_f32_row_does_not_depend_on_the_batch():
    torch.manual_seed(3)
    a, w = torch.randn(77, 300, device=DEV), torch.randn(91, 300, device=DEV)
    full = torch.empty(77, 91, device=DEV)
    ops().gemm_f32(a, w, full)
    one = torch.empty(1, 91, device=DEV)
    ops().gemm_f32(a[40:41].contiguous(), w, one)
    assert torch.equal(full[40], one[0])


# ------------------------------------------------------------------------------ paged cache helpers
def paged_from_dense(k, v, page_size, num_pages, dtype, seed=0):
    """k, v: lists (one per sequence) of [n, NKV, D].  Returns pages and a block table with
    the physical pages shuffled, so that logical order never equals physical order."""
    rng = random.Random(seed)
    nkv, d = k[0].shape[1], k[0].shape[2]
    pages = torch.full((num_pages, 2, nkv, page_size, d), float("nan"), dtype=torch.float32)
    free = list(range(num_pages))
    rng.shuffle(free)
    width = max(-(-x.shape[0] // page_size) for x in k)
    table = torch.full((len(k), width), -1, dtype=torch.int32)
    for s, (ks, vs) in enumerate(zip(k, v)):
        for b in range(-(-ks.shape[0] // page_size)):
            p = free.pop()
            table[s, b] = p
            n = min(page_size, ks.shape[0] - b * page_size)
            pages[p, 0, :, :n] = ks[b * page_size:b * page_size + n].transpose(0, 1)
            pages[p, 1, :, :n] = vs[b * page_size:b * page_size + n].transpose(0, 1)
    return pages.to(dtype), table


def memory_hog(milliseconds=30):
    """Queues device-to-device copies of 1 GB on a second stream, about `milliseconds` of them: kernels launched on
    the current stream right after this call run beside a kernel that saturates the memory system, which stretches
    every wait inside them (a timing no quiet test sees).  Returns what must stay alive until the device is idle."""
    side = torch.cuda.Stream()
    a = torch.empty(1 << 30, dtype=torch.uint8, device=DEV)
    b = torch.empty_like(a)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(max(1, int(milliseconds / 0.35))):          # ~0.35 ms a copy at 6 TB/s of reads + writes
            b.copy_(a, non_blocking=True)
    return side, a, b


def run_attention(q_list, k_list, v_list, pos0_list, nh, nkv, d, window, dtype, page_size=16, num_pages=64, repeats=None,
                  hog=False):
    """Queries q_list[s] ([n_s, NH, D]) sit at positions pos0_list[s].. of sequence s whose
    keys are k_list[s].  `repeats`: run the same step that often and return every result, [repeats, T, NH * D];
    `hog`: beside a kernel that saturates the memory system (see memory_hog)."""
    pages, table = paged_from_dense(k_list, v_list, page_size, num_pages, dtype)
    q = torch.cat([x.reshape(x.shape[0], nh * d) for x in q_list]).to(dtype)
    positions = torch.cat([torch.arange(p, p + x.shape[0], dtype=torch.int32) for p, x in zip(pos0_list, q_list)])
    token_seq = torch.cat([torch.full((x.shape[0],), s, dtype=torch.int32) for s, x in enumerate(q_list)])
    out = torch.empty(q.shape, dtype=dtype, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    from microllm_rocm_b200.kernels import attention
    from microllm_rocm_b200.parts.base import StepContext
    ctx = StepContext(num_tokens=q.shape[0], num_seqs=len(q_list), token_ids=positions.to(DEV), positions=positions.to(DEV),
                      token_seq=token_seq.to(DEV),
                      seq_starts=torch.tensor(np.cumsum([0] + [x.shape[0] for x in q_list]), dtype=torch.int32).to(DEV),
                      seq_pos0=torch.tensor(list(pos0_list), dtype=torch.int32).to(DEV),
                      seq_lens=torch.tensor([p + x.shape[0] for p, x in zip(pos0_list, q_list)], dtype=torch.int32).to(DEV),
                      block_tables={},
                      state_slots=None, logit_rows=None, error_flag=flag,
                      seq_starts_host=[int(v) for v in np.cumsum([0] + [x.shape[0] for x in q_list])],
                      seq_pos0_host=list(pos0_list), max_new_tokens=max(x.shape[0] for x in q_list),
                      max_seq_len=max(p + x.shape[0] for p, x in zip(pos0_list, q_list)))
    q, pages, table = q.to(DEV), pages.to(DEV), table.to(DEV)
    if repeats:
        outs = torch.empty((repeats, *q.shape), dtype=dtype, device=DEV)
        torch.cuda.synchronize()
        keep = memory_hog() if hog else None
        for i in range(repeats):
            attention.paged_attention(q, pages, outs[i], ctx, table, nh, nkv, d, 1.0 / math.sqrt(d), window)
        assert int(flag.item()) == 0
        torch.cuda.synchronize()
        del keep
        return outs.float().cpu()
    attention.paged_attention(q, pages, out, ctx, table, nh, nkv, d, 1.0 / math.sqrt(d), window)
    assert int(flag.item()) == 0
    return out.float().cpu()


def plain_attention_rows(q, k, v, pos0, window):
    """Reference for queries at positions pos0.. over keys k (which include those positions)."""
    n = q.shape[0]
    full_q = torch.zeros(pos0 + n, q.shape[1], q.shape[2])
    full_q[pos0:] = q
    return plain.causal_gqa_attention(full_q, k[:pos0 + n], v[:pos0 + n], window)[pos0:]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d,window", [(4, 1, 16, None), (6, 2, 32, 32), (7, 7, 48, None), (12, 2, 128, 40),
                                             (5, 5, 80, 17), (3, 1, 256, None), (14, 2, 64, 33)])
def test_paged_attention_prompts_and_decodes_in_one_batch(dtype, nh, nkv, d, window):
    torch.manual_seed(nh * d)
    lens = [70, 33, 1, 129]          # cached tokens after the step
    news = [70, 1, 1, 20]            # whole prompt, decode token, first token, later portion
    ks = [torch.randn(n, nkv, d) for n in lens]
    vs = [torch.randn(n, nkv, d) for n in lens]
    qs = [torch.randn(n, nh, d) for n in news]
    if dtype == torch.bfloat16:
        ks, vs, qs = ([x.to(dtype).float() for x in y] for y in (ks, vs, qs))
    got = run_attention(qs, ks, vs, [l - n for l, n in zip(lens, news)], nh, nkv, d, window, dtype)
    want = torch.cat([plain_attention_rows(q, k, v, l - n, window).reshape(n, nh * d)
                      for q, k, v, l, n in zip(qs, ks, vs, lens, news)])
    assert torch.allclose(got, want, **tol(dtype)), float((got - want).abs().max())


@pytest.mark.parametrize("nh,nkv,d", [(12, 2, 128), (4, 4, 64), (6, 1, 64)])
def test_decode_step_of_long_and_short_sequences_shares_one_key_split(nh, nkv, d):
    """One decode step for sequences of 1,500, 20, 300 and 1 cached tokens: the number of CTAs that share a
    (sequence, kv head) is chosen for the longest, so the short sequences leave most of those CTAs without
    a single key tile; their empty shares must drop out of the merge."""
    torch.manual_seed(nh + d)
    lens = [1500, 20, 300, 1]
    ks = [torch.randn(n, nkv, d).bfloat16().float() for n in lens]
    vs = [torch.randn(n, nkv, d).bfloat16().float() for n in lens]
    qs = [torch.randn(1, nh, d).bfloat16().float() for _ in lens]
    got = run_attention(qs, ks, vs, [n - 1 for n in lens], nh, nkv, d, None, torch.bfloat16, num_pages=130)
    want = torch.cat([plain_attention_rows(q, k, v, n - 1, None).reshape(1, nh * d) for q, k, v, n in zip(qs, ks, vs, lens)])
    assert torch.isfinite(got).all()
    assert torch.allclose(got, want, **tol(torch.bfloat16)), float((got - want).abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_one_far_key_among_hundreds_dominates(dtype):
    """Query and one key far back are scaled so that their score stands out: the output must
    be (nearly) that key's value, which a kernel that drops or misplaces far keys cannot give."""
    torch.manual_seed(5)
    nh, nkv, d, n = 4, 2, 64, 700
    k, v = torch.randn(n, nkv, d) * 0.1, torch.randn(n, nkv, d)
    q = torch.randn(1, nh, d) * 0.1
    far = 3                                             # sits in the first page
    direction = torch.randn(d)
    direction /= direction.norm()
    q[0, :] = direction * 30
    k[far, :] = direction * 30
    if dtype == torch.bfloat16:
        k, v, q = (x.to(dtype).float() for x in (k, v, q))
    got = run_attention([q], [k], [v], [n - 1], nh, nkv, d, None, dtype).reshape(nh, d)
    for h in range(nh):
        assert torch.allclose(got[h], v[far, h // 2], atol=3e-2 if dtype == torch.bfloat16 else 1e-4)
    # with a window that ends one key short of it, the far key must be invisible
    got_w = run_attention([q], [k], [v], [n - 1], nh, nkv, d, n - 1 - far, dtype).reshape(nh, d)
    want_w = plain_attention_rows(q, k, v, n - 1, n - 1 - far).reshape(nh, d)
    assert torch.allclose(got_w, want_w, **tol(dtype))
    assert not torch.allclose(got_w[0], v[far, 0], atol=0.2)
    # and with a window that just reaches it, visible again
    got_in = run_attention([q], [k], [v], [n - 1], nh, nkv, d, n - far, dtype).reshape(nh, d)
    assert torch.allclose(got_in[0], v[far, 0], atol=3e-2 if dtype == torch.bfloat16 else 1e-4)


@pytest.mark.parametrize("nh,nkv,d,window,page_size", [(12, 2, 128, None, 16), (6, 2, 128, 200, 16), (4, 4, 64, None, 32),
                                                        (5, 1, 64, 129, 8), (2, 1, 128, 64, 128), (3, 3, 128, 1000, 64)])
def test_tcgen05_prompt_attention_beside_short_portions(nh, nkv, d, window, page_size):
    """Long prompt portions go through the tcgen05 kernel (128-row tiles, 128-key tiles), short ones
    and decoded tokens through the mma.sync kernel, in one step.  Portions start at positions that
    are no multiple of the tile, end inside a page, and unused slots of the pages hold NaN."""
    torch.manual_seed(nh * d + page_size)
    lens = [300, 517, 90, 131, 256]          # cached tokens after the step
    news = [300, 440, 1, 20, 128]            # whole prompt, later portion, decode token, short portion, exact tile
    ks = [torch.randn(n, nkv, d).bfloat16().float() for n in lens]
    vs = [torch.randn(n, nkv, d).bfloat16().float() for n in lens]
    qs = [torch.randn(n, nh, d).bfloat16().float() for n in news]
    pages_needed = sum(-(-n // page_size) for n in lens) + 3
    got = run_attention(qs, ks, vs, [l - n for l, n in zip(lens, news)], nh, nkv, d, window, torch.bfloat16,
                        page_size=page_size, num_pages=pages_needed)
    want = torch.cat([plain_attention_rows(q, k, v, l - n, window).reshape(n, nh * d)
                      for q, k, v, l, n in zip(qs, ks, vs, lens, news)])
    assert torch.isfinite(got).all()
    assert torch.allclose(got, want, **tol(torch.bfloat16)), float((got - want).abs().max())


def test_tcgen05_prompt_attention_far_key_and_window_edge():
    """In a 700-token prompt every query from 400 on is aligned with key 3 (five key tiles back) so that
    its score stands out; the outputs must be that key's value.  A window that ends one key short of it
    for the last query only must hide it from that query alone."""
    torch.manual_seed(11)
    nh, nkv, d, n = 4, 2, 128, 700
    k, v = torch.randn(n, nkv, d) * 0.1, torch.randn(n, nkv, d)
    q = torch.randn(n, nh, d) * 0.1
    far = 3
    direction = torch.randn(d)
    direction /= direction.norm()
    q[400:, :] = direction * 30
    k[far, :] = direction * 30
    k, v, q = (x.bfloat16().float() for x in (k, v, q))
    got = run_attention([q], [k], [v], [0], nh, nkv, d, None, torch.bfloat16, num_pages=50).reshape(n, nh, d)
    for h in range(nh):
        assert torch.allclose(got[400:, h], v[far, h // 2].expand(n - 400, d), atol=3e-2)
    window = n - 1 - far                      # the last query sees keys far+1..n-1, the one before it sees `far`
    got_w = run_attention([q], [k], [v], [0], nh, nkv, d, window, torch.bfloat16, num_pages=50).reshape(n, nh, d)
    want_w = plain_attention_rows(q, k, v, 0, window)
    assert torch.allclose(got_w, want_w, **tol(torch.bfloat16)), float((got_w - want_w).abs().max())
    assert torch.allclose(got_w[n - 2, 0], v[far, 0], atol=3e-2)
    assert not torch.allclose(got_w[n - 1, 0], v[far, 0], atol=0.2)


def test_tcgen05_prompt_attention_when_one_softmax_warp_has_more_to_do():
    """The last 32 rows of every 128-row tile are aligned with keys that grow from key tile to key tile, so that
    their maxima outgrow the rescale threshold at EVERY tile and their softmax warp has the accumulator to rescale
    each time, while the three other warps never do and run ahead.  Equal to the plain attention, the same bits
    every time.  (test_a_held_back_warp_changes_nothing pulls the warps apart by force.)"""
    got, want = lagging_rows_case()
    assert torch.allclose(got[0], want, **tol(torch.bfloat16)), float((got[0] - want).abs().max())
    assert torch.equal(got[0], got[1]) and torch.equal(got[0], got[2])


def lagging_rows_case(repeats=3):
    torch.manual_seed(17)
    nh, nkv, d, n = 8, 2, 128, 2048
    k, v = torch.randn(n, nkv, d) * 0.1, torch.randn(n, nkv, d)
    q = torch.randn(n, nh, d) * 0.1
    direction = torch.randn(d)
    direction /= direction.norm()
    tile = torch.arange(n) // 128
    k += direction * 9.0 * tile[:, None, None]                 # + 81 * 0.088 * log2(e) = 10 > 8 doublings per key tile
    lagging = (torch.arange(n) % 128) >= 96
    q[lagging] = direction * 9.0
    k, v, q = (x.bfloat16().float() for x in (k, v, q))
    want = plain_attention_rows(q, k, v, 0, None).reshape(n, nh * d)
    got = run_attention([q], [k], [v], [0], nh, nkv, d, None, torch.bfloat16, page_size=64, num_pages=40, repeats=repeats)
    assert torch.isfinite(got).all()
    return got, want


def served_size_cases(flag):
    """name -> a function that runs one of the warp-specialised kernels at a served size and returns its result."""
    from microllm_rocm_b200.kernels import attention, gemm_bf16
    from microllm_rocm_b200.parts.base import StepContext
    torch.manual_seed(31)

    def rand(*shape, scale=1.0):
        return (torch.randn(*shape, device=DEV) * scale).bfloat16()

    cases = {}
    x1, w1 = rand(64, 8960), rand(1536, 8960, scale=0.02)
    cases["stream_partials"] = lambda: gemm_bf16.stream_partials(x1, w1, error_flag=flag).clone()
    x2, w2 = rand(16, 1536), rand(30000, 1536, scale=0.02)                # more tiles than SMs: persistent CTAs, two accumulators
    cases["stream_many_tiles"] = lambda: gemm_bf16.stream_partials(x2, w2, error_flag=flag).clone()
    x3, w3 = rand(64, 3584), rand(2 * 18944, 3584, scale=0.02)

    def stream_silu():
        out = torch.empty(64, 18944, dtype=torch.bfloat16, device=DEV)
        gemm_bf16.stream_silu_mul(x3, w3, out, error_flag=flag)
        return out
    cases["stream_silu"] = stream_silu
    x4, w4 = rand(2048, 3584), rand(4608, 3584, scale=0.02)

    def pair():
        out = torch.empty(2048, 4608, dtype=torch.bfloat16, device=DEV)
        gemm_bf16.gemm_pair(x4, w4, out, error_flag=flag)
        return out
    cases["pair"] = pair
    x5, w5 = rand(2048, 1536), rand(2 * 8960, 1536, scale=0.02)

    def pair_dual():
        out = torch.empty(2048, 8960, dtype=torch.bfloat16, device=DEV)
        gemm_bf16.gemm_pair(x5, w5, out, dual_rows=8960, error_flag=flag)
        return out
    cases["pair_dual"] = pair_dual
    x6 = rand(8, 1536)

    def gemv():
        out = torch.empty(8, 8960, dtype=torch.bfloat16, device=DEV)
        gemm_bf16.gemv_silu_mul(x6, w5, out)
        return out
    cases["gemv"] = gemv

    nh, nkv, d, batch, context = 28, 4, 128, 64, 2100
    pages_per_seq = -(-context // 64)
    pages = rand(batch * pages_per_seq + 1, 2, nkv, 64, d)
    table = torch.randperm(batch * pages_per_seq, device=DEV).int().view(batch, pages_per_seq)
    q = rand(batch, nh * d)
    lens = [context - 7 * (i % 5) for i in range(batch)]
    ints = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    ctx = StepContext(num_tokens=batch, num_seqs=batch, token_ids=ints([0] * batch), positions=ints([n - 1 for n in lens]),
                      token_seq=ints(list(range(batch))), seq_starts=ints(list(range(batch + 1))),
                      seq_pos0=ints([n - 1 for n in lens]), seq_lens=ints(lens), block_tables={}, state_slots=None,
                      logit_rows=None, error_flag=flag, seq_starts_host=list(range(batch + 1)),
                      seq_pos0_host=[n - 1 for n in lens], max_new_tokens=1, max_seq_len=max(lens))

    def decode(ring):
        def run():
            attention.DECODE_RING = ring
            try:
                out = torch.empty_like(q)
                attention.paged_attention(q, pages, out, ctx, table, nh, nkv, d, 1.0 / math.sqrt(d), None)
                return out
            finally:
                attention.DECODE_RING = None
        return run
    cases["decode_ring"] = decode(True)
    cases["decode_t"] = decode(False)
    return cases


@pytest.mark.parametrize("kernel", ["stream_partials", "stream_many_tiles", "stream_silu", "pair", "pair_dual", "gemv", "decode_ring",
                                    "decode_t"])
def test_kernels_with_barriers_or_rings_give_the_same_bits_beside_a_memory_hog(kernel):
    """The kernels that hand data from warp to warp through mbarriers or rings, at served sizes, twenty times in a row
    beside a kernel that saturates the memory system (every wait inside them is stretched, warps drift apart): each
    run must give the bits of the quiet run and raise no flag."""
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    run = served_size_cases(flag)[kernel]
    want = run()
    torch.cuda.synchronize()
    keep = memory_hog(40)
    got = [run() for _ in range(20)]
    torch.cuda.synchronize()
    del keep
    assert int(flag.item()) == 0
    assert torch.isfinite(want.float()).all()
    for i, g in enumerate(got):
        assert torch.equal(g, want), (kernel, i, float((g.float() - want.float()).abs().max()))


def held_back_builds():
    from microllm_rocm_b200.kernels import ops as o
    uses = {"attention_tc.cu": ["prompt"], "gemm_stream.cu": ["stream_partials", "stream_many_tiles", "stream_silu"],
            "gemm_tc2.cu": ["pair", "pair_dual"], "attention_mma.cu": ["decode_ring"]}
    return [(source, tuple(sorted(defines.items())), case) for source, defines in o.lagged_sources() for case in uses[source]]


@pytest.mark.parametrize("source,defines,case", held_back_builds())
def test_a_held_back_warp_changes_nothing(source, defines, case):
    """Every kernel whose warps have roles of their own (copy, MMA issue, epilogue or softmax) and meet at mbarriers is
    built once more per role with that role's warp sleeping 3 us at every turn of its loop (-DMLB_LAG_WARP, and
    -DMLB_LAG_RANK for the kernel of CTA pairs): the others then run as far ahead as the barriers let them.  A
    barrier that counts arrivals and can be completed by a fast warp's NEXT arrival in place of the slow warp's, a
    parity wait that can miss a phase, a buffer handed back too early: each shows as other bits or as a wait that
    runs out.  (The prompt attention kernel's single barrier for two P buffers did, with warp 2 or 5 held back.)"""
    from microllm_rocm_b200.kernels import ops as o
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    run = (lambda: lagging_rows_case(repeats=1)[0][0]) if case == "prompt" else served_size_cases(flag)[case]
    want = run()
    torch.cuda.synchronize()
    held = {k: v for k, v in defines if k.startswith("MLB_LAG")}
    o.TEST_DEFINES[source] = held
    try:
        got = run()
        torch.cuda.synchronize()
    finally:
        del o.TEST_DEFINES[source]
    assert int(flag.item()) == 0
    assert torch.equal(got, want), float((got.float() - want.float()).abs().max())


def test_prompt_portions_and_decoded_tokens_side_by_side_give_the_same_bits_every_time():
    """Three decoded tokens at 8,200 keys, the last 22 tokens of a prompt at 8,170 and the first 2,023 of another, with
    40 heads in 8 groups: the decoded tokens' kernel and the prompt portions' kernel run at the same time.  Thirty runs
    of the same step must agree bit for bit, and with the run in which the two kernels follow one another.  (In the
    22-row tile three of the four softmax warps work on rows of the NEXT sequence, so the warps of a CTA are out of
    step with one another; what the kernels compute is checked against the plain attention by the tests above.)"""
    from microllm_rocm_b200.kernels import attention
    torch.manual_seed(23)
    nh, nkv, d = 40, 8, 128
    lens = [8207, 8202, 8198, 8192, 2023]
    news = [1, 1, 1, 22, 2023]
    ks = [(torch.randn(n, nkv, d) * 0.5).bfloat16().float() for n in lens]
    vs = [torch.randn(n, nkv, d).bfloat16().float() for n in lens]
    qs = [torch.randn(n, nh, d).bfloat16().float() for n in news]
    pos0 = [l - n for l, n in zip(lens, news)]
    pages = sum(-(-n // 64) for n in lens) + 2
    attention.CONCURRENT_ATTENTION = False
    try:
        want = run_attention(qs, ks, vs, pos0, nh, nkv, d, None, torch.bfloat16, page_size=64, num_pages=pages)
    finally:
        attention.CONCURRENT_ATTENTION = True
    got = run_attention(qs, ks, vs, pos0, nh, nkv, d, None, torch.bfloat16, page_size=64, num_pages=pages, repeats=30, hog=True)
    assert torch.isfinite(got).all()
    for i in range(got.shape[0]):
        assert torch.equal(got[i], want), (i, float((got[i] - want).abs().max()))


@pytest.mark.parametrize("page_size", [4, 16, 64])
def test_window_and_page_edges(page_size):
    """Every query position around page edges and the window's edge, one token at a time."""
    torch.manual_seed(6)
    nh, nkv, d, W, n = 2, 1, 32, 2 * page_size, 3 * page_size + 3
    k, v, q = torch.randn(n, nkv, d), torch.randn(n, nkv, d), torch.randn(n, nh, d)
    want = plain.causal_gqa_attention(q, k, v, W)
    for pos in list(range(0, 3)) + list(range(page_size - 2, page_size + 2)) + list(range(W - 2, W + 3)) + [n - 1]:
        got = run_attention([q[pos:pos + 1]], [k[:pos + 1]], [v[:pos + 1]], [pos], nh, nkv, d, W, torch.float32,
                            page_size=page_size)
        assert torch.allclose(got.reshape(nh, d), want[pos], atol=2e-5), pos


# ------------------------------------------------------------------------------ rope + kv store
@pytest.mark.parametrize("kv_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d,rot,inter", [(4, 1, 16, 16, False), (6, 2, 32, 32, False), (3, 3, 128, 64, False),
                                                (2, 1, 48, 48, True), (5, 1, 256, 256, False)])
def test_rope_bias_and_paged_store(kv_dtype, nh, nkv, d, rot, inter):
    from microllm_rocm_b200.parts.rotary import inverse_frequencies
    torch.manual_seed(d + nh)
    T, page, theta = 23, 8, 1e6
    width = (nh + 2 * nkv) * d
    qkv, bias = torch.randn(T, width), torch.randn(width) * 0.3
    positions = torch.tensor([0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 100, 101, 40, 41, 42, 43, 44, 45, 46, 47, 48, 63, 64],
                             dtype=torch.int32)
    token_seq = torch.tensor([0] * 10 + [1] * 2 + [2] * 9 + [3] * 2, dtype=torch.int32)
    num_pages, maxb = 40, 16
    table = torch.full((4, maxb), -1, dtype=torch.int32)
    perm = list(range(num_pages))
    random.Random(1).shuffle(perm)
    for s_, p_ in sorted({(s_, int(p_) // page) for s_, p_ in zip(token_seq.tolist(), positions.tolist())}):
        table[s_, p_] = perm.pop()
    pages = torch.zeros(num_pages, 2, nkv, page, d, dtype=kv_dtype, device=DEV)
    q_out = torch.empty(T, nh * d, dtype=kv_dtype, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    inv = torch.from_numpy(inverse_frequencies(theta, rot)).to(DEV)
    ops().rope_kv_write(qkv.to(DEV), bias.to(DEV), positions.to(DEV), token_seq.to(DEV), table.to(DEV), inv, rot, inter,
                        q_out, pages, nh, nkv, d, flag)
    assert int(flag.item()) == 0
    x = (qkv + bias).view(T, nh + 2 * nkv, d)

    def rotate(heads):                  # plain rotation of the first `rot` elements
        part = heads[..., :rot]
        if inter:
            part = torch.cat([part[..., 0::2], part[..., 1::2]], -1)
        # frequencies of a rotary width `rot`
        half = rot // 2
        i = np.arange(half, dtype=np.float32)
        invf = np.power(np.float32(theta), (np.float32(-2.0) * i) / np.float32(rot), dtype=np.float32)
        out = part.clone()
        for t in range(T):
            ang = np.float32(positions[t].item()) * invf
            c, s = torch.from_numpy(np.cos(ang)), torch.from_numpy(np.sin(ang))
            a, b = part[t, :, :half], part[t, :, half:]
            out[t, :, :half], out[t, :, half:] = a * c - b * s, a * s + b * c
        if inter:
            re = torch.empty_like(out)
            re[..., 0::2], re[..., 1::2] = out[..., :half], out[..., half:]
            out = re
        return torch.cat([out, heads[..., rot:]], -1)

    if rot == d and not inter:          # the model's own case: also against the plain implementation
        assert torch.allclose(rotate(x[:, :nh]), plain.rope_split_half(x[:, :nh], positions.tolist(), theta), atol=1e-6)
    want_q, want_k, want_v = rotate(x[:, :nh]), rotate(x[:, nh:nh + nkv]), x[:, nh + nkv:]
    t_ = tol(kv_dtype)
    assert torch.allclose(q_out.float().cpu().view(T, nh, d), want_q, **t_)
    pc = pages.float().cpu()
    for t in range(T):
        p = table[token_seq[t], positions[t] // page]
        slot = positions[t] % page
        assert torch.allclose(pc[p, 0, :, slot], want_k[t], **t_)
        assert torch.allclose(pc[p, 1, :, slot], want_v[t], **t_)
    # nothing else was touched
    written = torch.zeros(num_pages, page, dtype=torch.bool)
    for t in range(T):
        written[table[token_seq[t], positions[t] // page], positions[t] % page] = True
    assert (pc[:, :, :, :, :].abs().sum(dim=(1, 2, 4))[~written] == 0).all()


def test_rope_kv_write_refuses_to_write_without_a_page():
    from microllm_rocm_b200.parts.rotary import inverse_frequencies
    nh, nkv, d = 2, 1, 16
    qkv = torch.randn(2, (nh + 2 * nkv) * d, device=DEV)
    table = torch.tensor([[0, -1]], dtype=torch.int32, device=DEV)           # block 1 has no page
    pages = torch.zeros(2, 2, nkv, 4, d, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    q = torch.empty(2, nh * d, device=DEV)
    ops().rope_kv_write(qkv, None, torch.tensor([3, 4], dtype=torch.int32, device=DEV),
                        torch.zeros(2, dtype=torch.int32, device=DEV), table,
                        torch.from_numpy(inverse_frequencies(1e4, d)).to(DEV), d, False, q, pages, nh, nkv, d, flag)
    assert int(flag.item()) == 1
    assert pages[1].abs().sum() == 0, "page 1 belongs to someone else and must stay untouched"


# ------------------------------------------------------------------------------ selection
@pytest.mark.parametrize("vocab", [1003, 151936, 20000])
def test_argmax_ties_and_non_finite(vocab):
    """Small vocabularies go through one block per row, large ones through several blocks per row that
    meet at a ticket: ties across slices, the very last element, and non-finite values far from the maximum."""
    torch.manual_seed(vocab)
    x = torch.randn(7, vocab)
    x[0, 7] = x[0, vocab - 500] = 50.0                 # tie, possibly in different slices: the smaller index wins
    x[1, vocab - 1] = 60.0                             # last element
    x[2, vocab // 2 + 10] = float("nan")
    x[3, 0] = float("inf")
    x[5, vocab - 3] = float("-inf")                    # not finite, though far from the maximum
    x[6, 9000 % vocab] = x[6, 8191 % vocab] = x[6, 8192 % vocab] = 70.0    # ties on both sides of a slice edge
    out = torch.full((7,), -7, dtype=torch.int32, device=DEV)
    for _ in range(3):                                 # the tickets must be left ready for the next launch
        ops().argmax_rows(x.to(DEV), out)
        assert out.tolist() == [7, vocab - 1, -1, -1, int(x[4].argmax()), -1, min(9000 % vocab, 8191 % vocab, 8192 % vocab)]


@pytest.mark.parametrize("vocab", [97, 1003, 40000])
def test_sampling_kernel_matches_the_plain_sampler(vocab):
    torch.manual_seed(vocab)
    rows = 24
    x = torch.randn(rows, vocab) * 2
    x[3, 5] = x[3, 9] = x[3].max() + 1                 # ties at the top-k edge
    temps = [0.0, 0.8, 1.0, 0.8, 0.3, 2.0] * 4
    topk = [0, 0, 1, 2, 5, min(50, vocab)] * 4
    seeds = [7, 7, 7, 11, 12345678901234, 3] * 4
    draws = list(range(rows))
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops().sample_rows(x.to(DEV), torch.tensor(temps).to(DEV), torch.tensor(topk, dtype=torch.int32).to(DEV),
                      torch.tensor(seeds, dtype=torch.int64).to(DEV), torch.tensor(draws, dtype=torch.int64).to(DEV), out)
    want = [plain.sample_token(x[r].numpy(), temps[r], topk[r], seeds[r], draws[r]) for r in range(rows)]
    assert out.tolist() == want


def test_sampling_kernel_follows_the_distribution():
    logits = torch.tensor([[0.0, 1.0, 2.0, 0.5, -1.0]]).repeat(4000, 1)
    out = torch.empty(4000, dtype=torch.int32, device=DEV)
    ops().sample_rows(logits.to(DEV), torch.full((4000,), 0.8).to(DEV), torch.zeros(4000, dtype=torch.int32).to(DEV),
                      torch.full((4000,), 7, dtype=torch.int64).to(DEV), torch.arange(4000, dtype=torch.int64).to(DEV), out)
    p = torch.softmax(logits[0] / 0.8, 0)
    freq = torch.bincount(out.cpu().long(), minlength=5) / 4000.0
    assert (freq - p).abs().max() < 0.03


def test_kernels_refuse_bad_sizes_with_a_clear_error():
    from microllm_rocm_b200.kernels.build import KernelError
    with pytest.raises(KernelError, match="no CPU path"):
        ops().rmsnorm(torch.randn(2, 4), torch.randn(4), 1e-5, torch.empty(2, 4))
    with pytest.raises(KernelError, match="shapes"):
        ops().gemm_f32(torch.randn(2, 4, device=DEV), torch.randn(3, 5, device=DEV), torch.empty(2, 3, device=DEV))
    from microllm_rocm_b200.kernels import attention
    with pytest.raises(KernelError, match="head_dim"):
        attention.check_head_dim(264)
    with pytest.raises(KernelError, match="head_dim"):
        attention.check_head_dim(17)


def test_scatter_int_and_pinned_uploads():
    """The two small helpers of steps issued ahead: selected tokens go to their places in the next step's input
    (indices outside either array are skipped, nothing else is touched), and small arrays reach the device through
    pinned slots, many more of them than the ring has slots, with their values intact."""
    o = ops()
    dst = torch.full((10,), -7, dtype=torch.int32, device=DEV)
    src = torch.arange(100, 106, dtype=torch.int32, device=DEV)
    to = o.upload([0, 9, 4, 12, -1, 3], "int32", torch.device(DEV))
    frm = o.upload([5, 0, 2, 1, 1, 77], "int32", torch.device(DEV))
    o.scatter_int(dst, to, src, frm)
    assert dst.tolist() == [105, -7, -7, -7, 102, -7, -7, -7, -7, 100]
    kept = []
    for i in range(100):                       # three times round the ring, while earlier copies may still be queued
        values = [i * 1000 + j for j in range(1 + i % 7)]
        kept.append((values, o.upload(values, "int64", torch.device(DEV))))
    floats = o.upload([0.5, -1.25], "float32", torch.device(DEV))
    big = o.upload(list(range(40000)), "int32", torch.device(DEV))        # larger than a slot
    torch.cuda.synchronize()
    assert all(t.tolist() == v for v, t in kept) and floats.tolist() == [0.5, -1.25] and big[-1].item() == 39999
    assert o.upload([], "int32", torch.device(DEV)).numel() == 0


# ------------------------------------------------------------------------------ tcgen05 products
@pytest.mark.parametrize("M,N,K,splits,stages", [
    (9, 2048, 1536, None, 0), (16, 1536, 8960, None, 0), (33, 1000, 264, 2, 0), (64, 1536, 8960, None, 0),
    (64, 384, 192, 3, 2), (128, 130, 72, 1, 0), (100, 19000, 1536, None, 3), (17, 200, 8, None, 0), (1, 128, 64, 1, 0),
    (64, 17920, 1536, 1, 0), (48, 2500, 1000, 7, 2)])
def test_stream_partials_sum_to_the_product(M, N, K, splits, stages):
    """The tcgen05 weight-streaming product at 1..128 tokens: widths and K that are no multiple of the tile, K cut
    into ranges of uneven length, a ring of two or three stages that wraps many times, and more row tiles than
    SMs (each CTA then walks several tiles with its accumulator double-buffered).  The partial results, added in
    split order, are the product; a second call gives the same bits."""
    from microllm_rocm_b200.kernels import gemm_bf16
    torch.manual_seed(M + N + K)
    x = torch.randn(M, K).bfloat16().to(DEV)
    w = torch.randn(N, K).bfloat16().to(DEV)
    bias = torch.randn(N, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert gemm_bf16.stream_supported(x, w)
    part = gemm_bf16.stream_partials(x, w, bias, splits=splits, stages=stages, error_flag=flag)
    assert part.dim() == 3 and part.shape[1:] == (M, N) and (splits is None or part.shape[0] <= splits)
    again = gemm_bf16.stream_partials(x, w, bias, splits=splits, stages=stages, error_flag=flag)
    assert int(flag.item()) == 0
    assert torch.equal(part, again)
    got = part[0].double()
    for i in range(1, part.shape[0]):
        got += part[i].double()
    want = x.double() @ w.double().t() + bias.double()
    assert (got - want).abs().max().item() <= 2e-5 * math.sqrt(K) * 4, float((got - want).abs().max())


@pytest.mark.parametrize("M,I,K,stages", [(64, 1120, 1536, 0), (9, 176, 64, 0), (33, 520, 192, 2), (128, 2240, 1536, 0),
                                          (100, 9600, 192, 3), (16, 8960, 1536, 0), (17, 23, 40, 0)])
def test_stream_silu_mul(M, I, K, stages):
    """Gate/up with the activation as the epilogue: 64 gate rows stacked on 64 up rows per tile, the halves
    exchanged through shared memory; token counts that end inside a 16- and a 32-token chunk, an intermediate
    size that ends inside a tile, and more tiles than SMs."""
    from microllm_rocm_b200.kernels import gemm_bf16
    torch.manual_seed(I + M)
    x = (torch.randn(M, K) * 0.5).bfloat16()
    w = (torch.randn(2 * I, K) * 0.2).bfloat16()
    w[0, :] = x[0].float() * 4                           # one large positive and one large negative gate value:
    w[1, :] = -x[0].float() * 4                          # both branches of the sigmoid
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    gemm_bf16.stream_silu_mul(x.to(DEV), w.to(DEV), out, stages=stages, error_flag=flag)
    assert int(flag.item()) == 0
    want = plain.swiglu(x.float() @ w[:I].float().t(), x.float() @ w[I:].float().t())
    got = out.float().cpu()
    assert torch.isfinite(got).all()
    assert torch.allclose(got, want, atol=2e-2, rtol=2e-2), float((got - want).abs().max())


def test_stream_product_refuses_what_it_cannot_take():
    from microllm_rocm_b200.kernels import gemm_bf16
    from microllm_rocm_b200.kernels.build import KernelError
    x, w = torch.randn(12, 20, device=DEV).bfloat16(), torch.randn(8, 20, device=DEV).bfloat16()
    assert not gemm_bf16.stream_supported(x, w)                       # K is no multiple of 8: TMA cannot address it
    with pytest.raises(KernelError, match="multiples of 8"):
        gemm_bf16.stream_partials(x, w)
    # the dispatcher sends such a product to the library instead of failing
    y = gemm_bf16.linear_bf16(x, w, None, torch.float32, None, partials_ok=True)
    assert y.dim() == 2 and torch.allclose(y.cpu(), x.float().cpu() @ w.float().cpu().t(), atol=1e-2)
    big = torch.randn(129, 64, device=DEV).bfloat16()
    with pytest.raises(KernelError, match="1..128"):
        gemm_bf16.stream_partials(big, torch.randn(8, 64, device=DEV).bfloat16())


@pytest.mark.parametrize("M,N,K,out_dtype", [(256, 256, 64, torch.float32), (2048, 1536, 1536, torch.float32),
                                             (300, 520, 200, torch.bfloat16), (1000, 2048, 1536, torch.bfloat16),
                                             (129, 100, 72, torch.float32), (3000, 300, 4096, torch.bfloat16)])
def test_cta_pair_product_against_fp32(M, N, K, out_dtype):
    """tcgen05.mma.cta_group::2: sizes that are no multiple of the 256 x 256 pair tile, more tiles than
    pairs (the double-buffered accumulator and the ring wrap around), with and without a bias."""
    from microllm_rocm_b200.kernels import gemm_bf16
    torch.manual_seed(M + N + K)
    x, w, bias = (torch.randn(M, K) * 0.5).bfloat16(), (torch.randn(N, K) * 0.5).bfloat16(), torch.randn(N)
    want = x.double() @ w.double().t() + bias.double()
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    gemm_bf16.gemm_pair(x.to(DEV), w.to(DEV), out, bias=bias.to(DEV))
    assert int(gemm_bf16.error_flag(torch.device(DEV)).item()) == 0
    got = out.double().cpu()
    tol_ = 2e-5 * math.sqrt(K) * 4 if out_dtype == torch.float32 else 2e-2 * want.abs().max().item()
    assert (got - want).abs().max() <= tol_, float((got - want).abs().max())
    if out_dtype == torch.float32:                      # accumulate on top of what is there
        gemm_bf16.gemm_pair(x.to(DEV), w.to(DEV), out, accumulate=True)
        want2 = want + x.double() @ w.double().t()
        assert (out.double().cpu() - want2).abs().max() <= 2 * tol_


@pytest.mark.parametrize("M,I,K", [(2048, 1120, 1536), (130, 176, 64), (700, 520, 192)])
def test_cta_pair_dual_product_silu_mul(M, I, K):
    from microllm_rocm_b200.kernels import gemm_bf16
    torch.manual_seed(I + M)
    x = (torch.randn(M, K) * 0.5).bfloat16()
    w = (torch.randn(2 * I, K) * 0.2).bfloat16()
    out = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    gemm_bf16.gemm_pair(x.to(DEV), w.to(DEV), out, dual_rows=I)
    want = plain.swiglu(x.float() @ w[:I].float().t(), x.float() @ w[I:].float().t())
    assert torch.allclose(out.float().cpu(), want, atol=2e-2, rtol=2e-2), float((out.float().cpu() - want).abs().max())
    assert int(gemm_bf16.error_flag(torch.device(DEV)).item()) == 0


@pytest.mark.parametrize("M,N,K,out_dtype", [(2048, 1536, 8960, torch.float32), (300, 520, 136, torch.bfloat16),
                                             (17, 2048, 1536, torch.float32), (1, 72, 40, torch.float32),
                                             (700, 17920, 1536, torch.bfloat16)])
def test_library_product_called_directly(M, N, K, out_dtype):
    """cuBLASLt through the package's own C entry point (no tensor framework in between): against fp32,
    into a given output with a row pitch of its own, and the same bits as a second call."""
    from microllm_rocm_b200.kernels import gemm_bf16
    torch.manual_seed(M + N)
    x, w = (torch.randn(M, K) * 0.5).bfloat16().to(DEV), (torch.randn(N, K) * 0.5).bfloat16().to(DEV)
    assert gemm_bf16._direct_library(torch.device(DEV))
    before = gemm_bf16.LaunchCounter.library
    y = gemm_bf16.library_linear(x, w, None, out_dtype, None)
    assert gemm_bf16.LaunchCounter.library == before + 1 and y.dtype == out_dtype and y.shape == (M, N)
    want = x.double().cpu() @ w.double().cpu().t()
    tol_ = 2e-5 * math.sqrt(K) * 4 if out_dtype == torch.float32 else 1e-2 * want.abs().max().item()
    assert (y.double().cpu() - want).abs().max() <= tol_
    wide = torch.full((M, N + 8), 7.0, dtype=out_dtype, device=DEV)
    gemm_bf16.library_linear(x, w, None, out_dtype, wide[:, :N])
    assert torch.equal(wide[:, :N], y) and float(wide[:, N:].float().min()) == 7.0


# ------------------------------------------------------------------------------ few-token weight streaming
@pytest.mark.parametrize("M,N,K", [(1, 64, 32), (8, 2048, 1536), (8, 1536, 8960), (3, 200, 96), (16, 384, 192),
                                   (9, 1000, 1024), (5, 70, 4096), (4, 9616, 96), (11, 12000, 160), (2, 1536, 8960)])
def test_gemv_partials_sum_to_the_product(M, N, K):
    from microllm_rocm_b200.kernels import gemm_bf16
    torch.manual_seed(M * 7 + N + K)
    x, w, bias = torch.randn(M, K).bfloat16(), torch.randn(N, K).bfloat16(), torch.randn(N)
    assert gemm_bf16.gemv_supported(x.to(DEV), w.to(DEV))
    part = gemm_bf16.gemv_partials(x.to(DEV), w.to(DEV), bias.to(DEV))
    assert part.dim() == 3 and part.shape[1:] == (M, N)
    want = x.double() @ w.double().t() + bias.double()
    got = part.double().sum(0).cpu()
    assert (got - want).abs().max() <= 2e-5 * math.sqrt(K) * 4
    # the consumers add the partial results up: residual += sum, then norm
    res = torch.randn(M, N)
    wn = 1 + 0.1 * torch.randn(N)
    r = res.to(DEV).clone()
    out = torch.empty(M, N, device=DEV)
    ops().add_rmsnorm(r, part, wn.to(DEV), 1e-6, out)
    assert torch.allclose(r.cpu().double(), res.double() + want, atol=2e-5 * math.sqrt(K) * 4)
    assert torch.allclose(out.cpu(), plain.rms_norm((res.double() + want).float(), wn, 1e-6), atol=1e-3, rtol=1e-3)
    r2 = res.to(DEV).clone()
    ops().add_inplace(r2, part)
    assert torch.equal(r2, r)


@pytest.mark.parametrize("M,I,K", [(8, 1120, 1536), (2, 176, 64), (13, 512, 192), (1, 1000, 96), (16, 72, 4096), (7, 23, 32)])
def test_gemv_silu_mul(M, I, K):
    from microllm_rocm_b200.kernels import gemm_bf16
    torch.manual_seed(I + M)
    x = (torch.randn(M, K) * 0.5).bfloat16()
    w = (torch.randn(2 * I, K) * 0.2).bfloat16()
    out = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    gemm_bf16.gemv_silu_mul(x.to(DEV), w.to(DEV), out)
    want = plain.swiglu(x.float() @ w[:I].float().t(), x.float() @ w[I:].float().t())
    assert torch.allclose(out.float().cpu(), want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("M,nh,nkv,d,K,rotate,with_bias", [(8, 12, 2, 128, 1536, True, True), (1, 4, 1, 16, 64, True, False),
                                                         (13, 5, 5, 48, 160, True, True), (16, 3, 1, 256, 96, False, True),
                                                         (3, 14, 2, 64, 896, True, True)])
def test_gemv_qkv_rope_projects_rotates_and_stores(M, nh, nkv, d, K, rotate, with_bias):
    """Projection, bias, split-half rotation and the paged store in one kernel, against the plain
    functions; tokens of three sequences at positions around page edges, pages in shuffled order."""
    from microllm_rocm_b200.kernels import gemm_bf16
    from microllm_rocm_b200.parts.rotary import inverse_frequencies
    torch.manual_seed(M + nh + d)
    theta, page = 1e6, 8
    width = (nh + 2 * nkv) * d
    x = (torch.randn(M, K) * 0.5).bfloat16()
    w = (torch.randn(width, K) * 0.1).bfloat16()
    bias = torch.randn(width) * 0.3 if with_bias else None
    positions = torch.tensor(([0, 7, 8, 100, 101, 40, 41, 63, 64, 15, 16, 17, 300, 301, 302, 303])[:M], dtype=torch.int32)
    token_seq = torch.tensor(([0, 0, 0, 1, 1, 2, 2, 2, 2, 0, 0, 0, 1, 1, 1, 1])[:M], dtype=torch.int32)
    num_pages, maxb = 64, 40
    table = torch.full((3, maxb), -1, dtype=torch.int32)
    perm = list(range(num_pages))
    random.Random(2).shuffle(perm)
    for s_, b_ in sorted({(s_, int(p_) // page) for s_, p_ in zip(token_seq.tolist(), positions.tolist())}):
        table[s_, b_] = perm.pop()
    pages = torch.zeros(num_pages, 2, nkv, page, d, dtype=torch.bfloat16, device=DEV)
    q_out = torch.empty(M, nh * d, dtype=torch.bfloat16, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    inv = torch.from_numpy(inverse_frequencies(theta, d)).to(DEV) if rotate else None
    assert gemm_bf16.gemv_fused_supported(x.to(DEV), w.to(DEV))
    gemm_bf16.gemv_qkv_rope(x.to(DEV), w.to(DEV), bias.to(DEV) if with_bias else None, positions.to(DEV), token_seq.to(DEV),
                            table.to(DEV), inv, q_out, pages, nh, nkv, d, flag)
    assert int(flag.item()) == 0
    y = x.float() @ w.float().t()
    if with_bias:
        y = y + bias
    y = y.view(M, nh + 2 * nkv, d)
    rot = (lambda h: plain.rope_split_half(h, positions.tolist(), theta)) if rotate else (lambda h: h)
    want_q, want_k, want_v = rot(y[:, :nh]), rot(y[:, nh:nh + nkv]), y[:, nh + nkv:]
    t_ = tol(torch.bfloat16)
    assert torch.allclose(q_out.float().cpu().view(M, nh, d), want_q, **t_)
    pc = pages.float().cpu()
    written = torch.zeros(num_pages, page, dtype=torch.bool)
    for t in range(M):
        p_, slot = table[token_seq[t], positions[t] // page], positions[t] % page
        assert torch.allclose(pc[p_, 0, :, slot], want_k[t], **t_)
        assert torch.allclose(pc[p_, 1, :, slot], want_v[t], **t_)
        written[p_, slot] = True
    assert (pc.abs().sum(dim=(1, 2, 4))[~written] == 0).all()            # nothing else was touched
    # a token without a page raises the flag and writes nothing
    table[:] = -1
    pages.zero_()
    gemm_bf16.gemv_qkv_rope(x.to(DEV), w.to(DEV), None, positions.to(DEV), token_seq.to(DEV), table.to(DEV), inv, q_out,
                            pages, nh, nkv, d, flag)
    assert int(flag.item()) == 1 and float(pages.float().abs().sum()) == 0.0


def test_rope_table_gives_the_same_rotation_bit_for_bit():
    """The step-wide (cos, sin) table is made with the rotation kernel's own expressions: with it and
    without it the queries and the cache must be identical."""
    from microllm_rocm_b200.parts.rotary import inverse_frequencies
    torch.manual_seed(9)
    nh, nkv, d, T, page = 6, 2, 64, 300, 16
    width = (nh + 2 * nkv) * d
    qkv, bias = torch.randn(T, width, device=DEV), torch.randn(width, device=DEV)
    inv = torch.from_numpy(inverse_frequencies(1e6, d)).to(DEV)
    pos = torch.arange(1000, 1000 + T, dtype=torch.int32, device=DEV)
    seq = torch.zeros(T, dtype=torch.int32, device=DEV)
    table = torch.arange(90, dtype=torch.int32, device=DEV).flip(0).reshape(1, 90).contiguous()
    outs = []
    for use_table in (False, True):
        pages = torch.zeros(90, 2, nkv, page, d, dtype=torch.bfloat16, device=DEV)
        q = torch.empty(T, nh * d, dtype=torch.bfloat16, device=DEV)
        flag = torch.zeros(1, dtype=torch.int32, device=DEV)
        cs = ops().rope_table(pos, inv) if use_table else None
        ops().rope_kv_write(qkv, bias, pos, seq, table, inv, d, False, q, pages, nh, nkv, d, flag, cs)
        assert int(flag.item()) == 0
        outs.append((q.cpu(), pages.cpu()))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    assert float(outs[0][1].float().abs().sum()) > 0


def test_rope_kv_write_adds_partial_projections():
    from microllm_rocm_b200.parts.rotary import inverse_frequencies
    torch.manual_seed(4)
    nh, nkv, d, T = 4, 2, 32, 5
    width = (nh + 2 * nkv) * d
    parts = torch.randn(3, T, width)
    bias = torch.randn(width)
    inv = torch.from_numpy(inverse_frequencies(1e4, d)).to(DEV)
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    seq = torch.zeros(T, dtype=torch.int32, device=DEV)
    table = torch.tensor([[1, 0]], dtype=torch.int32, device=DEV)
    outs = []
    for src in (parts.to(DEV), parts.sum(0).to(DEV)):
        pages = torch.zeros(2, 2, nkv, 4, d, device=DEV)
        q = torch.empty(T, nh * d, device=DEV)
        flag = torch.zeros(1, dtype=torch.int32, device=DEV)
        ops().rope_kv_write(src, bias.to(DEV), pos, seq, table, inv, d, False, q, pages, nh, nkv, d, flag)
        outs.append((q.cpu(), pages.cpu()))
    assert torch.allclose(outs[0][0], outs[1][0], atol=1e-5) and torch.allclose(outs[0][1], outs[1][1], atol=1e-5)
